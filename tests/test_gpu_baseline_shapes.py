"""Parity with the float64 oracle at the benchmark configurations' own sizes.

The oracle cannot run whole tensors of these sizes (the phase tensor alone is
17 GB at batch 16 x d_inner 1024 x d_state 16 x 16384 steps), but every
channel (b, i) of the scan is independent of the others and every row of the
phase projection is independent of the other rows, so the GPU runs the full
problem and the oracle runs a SAMPLE of its channels in float64 on the CPU:

* scan core (phase tensor given): dense upstream gradient; y, the final state,
  dtheta, du, ddt, dz and the gradient of the initial state of the sampled
  channels are compared;
* drop-in operator (phase projection + scan) and the complex / positive-real /
  Mamba scans: the upstream gradient is non-zero on the sampled channels only,
  so that every gradient of the full-size GPU run - including the sums over
  all channels (dx, dx_bias, dB, dC, dD) and the projection adjoint du that
  mixes all channels - is determined by the sample and can be compared in full;
* a dense full-oracle case at one batch entry, d_inner 1024 / 2048 and a short
  sequence covers the adjoint contractions with every row contributing.

Tolerances are the benchmark's: forward abs 1e-5 + rel 1e-4, gradients rel 1e-3
(with an absolute floor of 1e-5 of the tensor's largest magnitude, 3e-5 at 16384
steps: see _gfloor); which branch of the parity rule each comparison passed by
is in the test summary.
"""
import math

import pytest
import torch
import torch.nn.functional as F

import aussm_b200
from aussm_b200.s6 import selective_scan_fn
from oracle import s6 as OS6
from oracle import unitary as O
from oracle import variants as OV
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu

CONFIG1 = (16, 1024, 16)          # batch, d_inner, d_state of the scaling sweep
CONFIG2 = (8, 2048, 16, 4096)     # the three-variant configuration


def _need(gib):
    free, _total = torch.cuda.mem_get_info()
    if free < gib * 2**30:
        pytest.skip(f"needs about {gib} GiB of device memory")


def _sample_channels(b, d, count=8):
    """(batch entry, channel) pairs spread over the tensor, first and last included."""
    pairs = [(0, 0), (b - 1, d - 1)]
    g = torch.Generator().manual_seed(b * 131 + d)
    while len(pairs) < count:
        p = (int(torch.randint(b, (1,), generator=g)), int(torch.randint(d, (1,), generator=g)))
        if p not in pairs:
            pairs.append(p)
    return pairs


def _gfloor(t, steps=0):
    """Absolute floor of the gradient tolerance: 1e-5 of the tensor's largest magnitude, or - for long
    sequences - the accuracy float32 can give a recurrence of `steps` steps at all: each step rounds at
    2^-24 relative to the running magnitude and the roundings add like a random walk, 2 eps sqrt(steps)
    (3e-5 at 16384 steps).  Elements far below the largest one (cancellations) are judged against this floor,
    everything else against rel 1e-3."""
    return max(1e-5, 2.4e-7 * math.sqrt(steps)) * float(t.abs().max()) + 1e-12


# ---------------------------------------------------------------------------
# scan core, configuration 1 at all four sequence lengths
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("l", [256, 1024, 4096, 16384])
def test_baseline_config1_scan_core_sampled_channels(l):
    b, d, n = CONFIG1
    _need(4.5 * 4 * b * d * n * l / 2**30 + 4)
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1000 + l)
    r = lambda *s: torch.randn(*s, generator=g, device=dev)
    theta = ((torch.rand(b, d, n, l, generator=g, device=dev) * 2 - 1) * math.pi).requires_grad_(True)
    u, z, gy = r(b, d, l).requires_grad_(True), r(b, d, l).requires_grad_(True), r(b, d, l)
    dt = F.softplus(r(b, d, l)).requires_grad_(True)
    par = dict(B_r=F.softplus(r(n) / math.sqrt(n)), B_theta=r(n) / math.sqrt(n),
               C_r=F.softplus(r(n) / math.sqrt(n)), C_theta=r(n) / math.sqrt(n))
    Dsk = r(d)
    h0_re, h0_im = r(b, d, n).requires_grad_(True), r(b, d, n).requires_grad_(True)
    gh_re, gh_im = r(b, d, n), r(b, d, n)
    y, h_re, h_im = aussm_b200.scan_unitary(theta, u, dt, z, par["B_r"], par["B_theta"], par["C_r"], par["C_theta"],
                                            Dsk, h0_re, h0_im)
    ((y * gy).sum() + (h_re * gh_re).sum() + (h_im * gh_im).sum()).backward()
    assert aussm_b200.device_status() == 0

    pairs = _sample_channels(b, d)
    bi = torch.tensor([p[0] for p in pairs], device=dev)
    ci = torch.tensor([p[1] for p in pairs], device=dev)
    pick = lambda t: t.detach()[bi, ci].unsqueeze(0).cpu()           # (1, sample, ...)
    got = dict(y=pick(y), h_re=pick(h_re), h_im=pick(h_im), theta=pick(theta.grad), u=pick(u.grad),
               dt=pick(dt.grad), z=pick(z.grad), h0_re=pick(h0_re.grad), h0_im=pick(h0_im.grad))
    src = dict(theta=pick(theta), u=pick(u), dt=pick(dt), z=pick(z), h0_re=pick(h0_re), h0_im=pick(h0_im),
               gy=pick(gy), gh_re=pick(gh_re), gh_im=pick(gh_im), D=Dsk[ci].cpu())
    del theta, y, u, dt, z
    torch.cuda.empty_cache()

    res = {}
    for tag, dtype, fn in (("t", torch.float64, O.scan_unitary_recurrence), ("r", torch.float32, O.scan_unitary_cumsum)):
        leaf = {k: src[k].to(dtype).clone().requires_grad_(True) for k in ("theta", "u", "dt", "z", "h0_re", "h0_im")}
        p = {k: v.cpu().to(dtype) for k, v in par.items()}
        yo, hr, hi = fn(leaf["theta"], leaf["u"], leaf["dt"], leaf["z"], p["B_r"], p["B_theta"], p["C_r"],
                        p["C_theta"], src["D"].to(dtype), leaf["h0_re"], leaf["h0_im"])
        ((yo * src["gy"].to(dtype)).sum() + (hr * src["gh_re"].to(dtype)).sum()
         + (hi * src["gh_im"].to(dtype)).sum()).backward()
        res[tag] = dict(y=yo.detach(), h_re=hr.detach(), h_im=hi.detach(), **{k: v.grad for k, v in leaf.items()})
    for k in ("y", "h_re", "h_im"):
        assert_parity(f"L{l} {k}", got[k], res["t"][k], res["r"][k])
    for k in ("theta", "u", "dt", "z", "h0_re", "h0_im"):
        assert_parity(f"L{l} grad_{k}", got[k], res["t"][k], res["r"][k], atol=_gfloor(res["t"][k], l), rtol=1e-3)


# ---------------------------------------------------------------------------
# drop-in operator: phase projection (K = d_inner) feeding the scan
# ---------------------------------------------------------------------------
def _dropin_inputs(b, d, n, l, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, device=dev)
    sc = 1.0 / math.sqrt(n)
    return dict(u=r(b, d, l), dt=F.softplus(r(b, d, l)), x=r(d, n, d) / math.sqrt(d),
                x_bias=(torch.rand(d, n, generator=g, device=dev) * 2 - 1) * math.pi,
                B=torch.complex(r(n) * sc, r(n) * sc), C=torch.complex(r(n) * sc, r(n) * sc), D=r(d), z=r(b, d, l),
                gy=r(b, d, l))


NAMES = ["u", "dt", "x", "x_bias", "B", "C", "D", "z"]


def _dropin_gpu(inp):
    a = [inp[k].clone().requires_grad_(True) for k in NAMES]
    y = aussm_b200.ssm_adaptive_interface(*a, unitary=True)
    (y * inp["gy"]).sum().backward()
    assert aussm_b200.device_status() == 0
    return y.detach(), {k: t.grad for k, t in zip(NAMES, a)}


def _dropin_oracle_on_sample(inp, batches, chans, dtype):
    """The operator restricted to the channels `chans` of the batch entries `batches`: their phases need
    all rows of u of those batch entries, nothing of the other channels."""
    cdt = torch.complex128 if dtype == torch.float64 else torch.complex64
    bs, cs = torch.tensor(batches), torch.tensor(chans)
    c = lambda t: t.detach().cpu()
    u = c(inp["u"])[bs].to(dtype).requires_grad_(True)                 # (nb, d, l): every row feeds the projection
    dt = c(inp["dt"])[bs][:, cs].to(dtype).requires_grad_(True)
    z = c(inp["z"])[bs][:, cs].to(dtype).requires_grad_(True)
    x = c(inp["x"])[cs].to(dtype).requires_grad_(True)                 # (nc, n, d)
    xb = c(inp["x_bias"])[cs].to(dtype).requires_grad_(True)
    B = c(inp["B"]).to(cdt).requires_grad_(True)
    C = c(inp["C"]).to(cdt).requires_grad_(True)
    D = c(inp["D"])[cs].to(dtype).requires_grad_(True)
    theta = O.phase_projection(u, x, xb)                               # (nb, nc, n, l)
    fn = O.scan_unitary_recurrence if dtype == torch.float64 else O.scan_unitary_cumsum
    y, _, _ = fn(theta, u[:, cs], dt, z, F.softplus(B.real), B.imag, F.softplus(C.real), C.imag, D)
    (y * c(inp["gy"])[bs][:, cs].to(dtype)).sum().backward()
    return y.detach(), dict(u=u.grad, dt=dt.grad, z=z.grad, x=x.grad, x_bias=xb.grad, B=B.grad, C=C.grad, D=D.grad)


def _compare_dropin_sample(tag, inp, y, grads, batches, chans):
    steps = inp["u"].shape[-1]
    bs, cs = torch.tensor(batches), torch.tensor(chans)
    y64, g64 = _dropin_oracle_on_sample(inp, batches, chans, torch.float64)
    y32, g32 = _dropin_oracle_on_sample(inp, batches, chans, torch.float32)
    c = lambda t: t.detach().cpu()
    assert_parity(f"{tag} y", c(y)[bs][:, cs], y64, y32)
    sel = dict(u=c(grads["u"])[bs], dt=c(grads["dt"])[bs][:, cs], z=c(grads["z"])[bs][:, cs], x=c(grads["x"])[cs],
               x_bias=c(grads["x_bias"])[cs], D=c(grads["D"])[cs], B=torch.view_as_real(c(grads["B"])),
               C=torch.view_as_real(c(grads["C"])))
    for k, got in sel.items():
        t64, t32 = g64[k], g32[k]
        if t64.is_complex():
            t64, t32 = torch.view_as_real(t64), torch.view_as_real(t32)
        assert_parity(f"{tag} grad_{k}", got, t64, t32, atol=_gfloor(t64, steps), rtol=1e-3)
    # nothing may leak into channels and batch entries that got no upstream gradient
    other_b = [i for i in range(inp["u"].shape[0]) if i not in batches]
    if other_b:
        ob = torch.tensor(other_b)
        for k in ("u", "dt", "z"):
            assert float(c(grads[k])[ob].abs().max()) == 0.0, k
    mask = torch.ones(inp["x"].shape[0], dtype=torch.bool)
    mask[cs] = False
    assert float(c(grads["x"])[mask].abs().max()) == 0.0
    assert float(c(grads["x_bias"])[mask].abs().max()) == 0.0


@pytest.mark.parametrize("l", [256, 1024, 4096, 16384])
def test_baseline_config1_dropin_sampled_channels(l):
    b, d, n = CONFIG1
    _need(3.0 * 4 * b * d * n * l / 2**30 + 12)
    inp = _dropin_inputs(b, d, n, l, 2000 + l, "cuda")
    batches, chans = [0, 7, b - 1], [0, 3, 511, d - 1]
    keep = torch.zeros(b, d, 1, device="cuda")
    for bb in batches:
        keep[bb, chans] = 1.0
    inp["gy"] = inp["gy"] * keep
    y, grads = _dropin_gpu(inp)
    _compare_dropin_sample(f"L{l}", inp, y, grads, batches, chans)


@pytest.mark.parametrize("d,l", [(1024, 1024), (2048, 512)])
def test_baseline_width_dropin_dense_one_batch_entry(d, l):
    """Dense upstream gradient, every row of the adjoint contractions contributing (K = d*n = 16384 / 32768
    for du, K = l for dx), against the full float64 oracle of one batch entry."""
    n = 16
    inp = _dropin_inputs(1, d, n, l, 3000 + d, "cuda")
    y, grads = _dropin_gpu(inp)
    c = lambda t: t.detach().cpu()
    outs = {}
    for tag, dtype in (("t", torch.float64), ("r", torch.float32)):
        cdt = torch.complex128 if dtype == torch.float64 else torch.complex64
        a = [c(inp[k]).to(cdt if inp[k].is_complex() else dtype).requires_grad_(True) for k in NAMES]
        yo = O.interface_unitary(*a, max_parallel_length=l, recurrence=(tag == "t"))
        (yo * c(inp["gy"]).to(dtype)).sum().backward()
        outs[tag] = (yo.detach(), {k: t.grad for k, t in zip(NAMES, a)})
    assert_parity(f"D{d} y", y, outs["t"][0], outs["r"][0])
    for k in NAMES:
        got, t64, t32 = grads[k], outs["t"][1][k], outs["r"][1][k]
        if t64.is_complex():
            got, t64, t32 = torch.view_as_real(got), torch.view_as_real(t64), torch.view_as_real(t32)
        assert_parity(f"D{d} grad_{k}", got, t64, t32, atol=_gfloor(t64, l), rtol=1e-3)


# ---------------------------------------------------------------------------
# configuration 2: unitary, complex, positive-real and Mamba scans at batch 8 x d_inner 2048 x 4096 steps
# ---------------------------------------------------------------------------
def test_baseline_config2_unitary_dropin_sampled_channels():
    b, d, n, l = CONFIG2
    _need(3.0 * 4 * b * d * n * l / 2**30 + 12)
    inp = _dropin_inputs(b, d, n, l, 4000, "cuda")
    batches, chans = [0, 3, b - 1], [0, 5, 1023, d - 1]
    keep = torch.zeros(b, d, 1, device="cuda")
    for bb in batches:
        keep[bb, chans] = 1.0
    inp["gy"] = inp["gy"] * keep
    y, grads = _dropin_gpu(inp)
    _compare_dropin_sample("C2", inp, y, grads, batches, chans)


@pytest.mark.parametrize("kind", ["complex", "preal"])
def test_baseline_config2_complex_scan_sampled_channels(kind):
    """Scan core of the complex / positive-real operators on given eigenvalue exponents: decay magnitude
    exp(-softplus(N(0,1))), phase U(-pi, pi) (complex) or none (positive real)."""
    b, d, n, l = CONFIG2
    _need(5.0 * 4 * b * d * n * l / 2**30 + 8)
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(5000 + len(kind))
    r = lambda *s: torch.randn(*s, generator=g, device=dev)
    cplx = kind == "complex"
    rho = (-F.softplus(r(b, d, n, l))).requires_grad_(True)
    theta = ((torch.rand(b, d, n, l, generator=g, device=dev) * 2 - 1) * math.pi).requires_grad_(True) if cplx else None
    u, z = r(b, d, l).requires_grad_(True), r(b, d, l).requires_grad_(True)
    dt = F.softplus(r(b, d, l)).requires_grad_(True)
    sc = 1.0 / math.sqrt(n)
    Br, Cr = (r(b, n, l) * sc).requires_grad_(True), (r(b, n, l) * sc).requires_grad_(True)
    Bi = (r(b, n, l) * sc).requires_grad_(True) if cplx else None
    Ci = (r(b, n, l) * sc).requires_grad_(True) if cplx else None
    Dsk = r(d).requires_grad_(True)
    pairs = _sample_channels(b, d)
    gy = torch.zeros(b, d, l, device=dev)
    for bb, cc in pairs:
        gy[bb, cc] = r(l)
    y = aussm_b200.scan_complex(rho, theta, u, dt, z, Br, Bi, Cr, Ci, Dsk)
    (y * gy).sum().backward()
    assert aussm_b200.device_status() == 0

    c = lambda t: t.detach().cpu()
    batches = sorted({p[0] for p in pairs})
    outs = {}
    for bb in batches:                                     # one oracle run per sampled batch entry
        cs = torch.tensor([p[1] for p in pairs if p[0] == bb])
        for tag, dtype in (("t", torch.float64), ("r", torch.float32)):
            leaf = dict(rho=c(rho)[bb:bb + 1][:, cs], u=c(u)[bb:bb + 1][:, cs], dt=c(dt)[bb:bb + 1][:, cs],
                        z=c(z)[bb:bb + 1][:, cs], Br=c(Br)[bb:bb + 1], Cr=c(Cr)[bb:bb + 1], D=c(Dsk)[cs])
            if cplx:
                leaf.update(theta=c(theta)[bb:bb + 1][:, cs], Bi=c(Bi)[bb:bb + 1], Ci=c(Ci)[bb:bb + 1])
            leaf = {k: v.to(dtype).clone().requires_grad_(True) for k, v in leaf.items()}
            Bc = torch.complex(leaf["Br"], leaf["Bi"]) if cplx else leaf["Br"]
            Cc = torch.complex(leaf["Cr"], leaf["Ci"]) if cplx else leaf["Cr"]
            yo = OV.scan_complex_ref(leaf["rho"], leaf.get("theta"), leaf["u"], leaf["dt"], leaf["z"], Bc, Cc, leaf["D"])
            (yo * c(gy)[bb:bb + 1][:, cs].to(dtype)).sum().backward()
            outs[(bb, tag)] = (yo.detach(), {k: v.grad for k, v in leaf.items()}, cs)
    for bb in batches:
        y64, g64, cs = outs[(bb, "t")]
        y32, g32, _ = outs[(bb, "r")]
        assert_parity(f"{kind} b{bb} y", c(y)[bb:bb + 1][:, cs], y64, y32)
        got = dict(rho=c(rho.grad)[bb:bb + 1][:, cs], u=c(u.grad)[bb:bb + 1][:, cs], dt=c(dt.grad)[bb:bb + 1][:, cs],
                   z=c(z.grad)[bb:bb + 1][:, cs], Br=c(Br.grad)[bb:bb + 1], Cr=c(Cr.grad)[bb:bb + 1], D=None)
        if cplx:
            got.update(theta=c(theta.grad)[bb:bb + 1][:, cs], Bi=c(Bi.grad)[bb:bb + 1], Ci=c(Ci.grad)[bb:bb + 1])
        for k, v in got.items():
            if v is None:
                continue
            assert_parity(f"{kind} b{bb} grad_{k}", v, g64[k], g32[k], atol=_gfloor(g64[k], l), rtol=1e-3)
    # dD sums over the batch: add the sampled entries' contributions
    dD64 = torch.zeros(d, dtype=torch.float64)
    dD32 = torch.zeros(d, dtype=torch.float32)
    for bb in batches:
        dD64[outs[(bb, "t")][2]] += outs[(bb, "t")][1]["D"]
        dD32[outs[(bb, "r")][2]] += outs[(bb, "r")][1]["D"]
    assert_parity(f"{kind} grad_D", c(Dsk.grad), dD64, dD32, atol=_gfloor(dD64, l), rtol=1e-3)


def test_baseline_config2_real_scan_sampled_channels():
    """The Mamba block's real selective scan (A = -exp(N(0,1)) per channel and state) at configuration 2.
    Its oracle is the published recurrence written from the math (the third-party package the reference
    calls is absent), so this pins the kernel to that restatement, not to the package."""
    b, d, n, l = CONFIG2
    _need(12)
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(6000)
    r = lambda *s: torch.randn(*s, generator=g, device=dev)
    sc = 1.0 / math.sqrt(n)
    t = dict(u=r(b, d, l), delta=r(b, d, l) * 0.5, A=-torch.exp(r(d, n)), B=r(b, n, l) * sc, C=r(b, n, l) * sc,
             D=r(d), z=r(b, d, l), delta_bias=r(d) * 0.5)
    keys = list(t)
    t = {k: v.requires_grad_(True) for k, v in t.items()}
    pairs = _sample_channels(b, d)
    gy = torch.zeros(b, d, l, device=dev)
    for bb, cc in pairs:
        gy[bb, cc] = r(l)
    y = selective_scan_fn(*[t[k] for k in keys], delta_softplus=True)
    (y * gy).sum().backward()
    assert aussm_b200.device_status() == 0
    c = lambda v: v.detach().cpu()
    batches = sorted({p[0] for p in pairs})
    acc = {tag: dict(A=torch.zeros(d, n, dtype=dt_), D=torch.zeros(d, dtype=dt_), delta_bias=torch.zeros(d, dtype=dt_))
           for tag, dt_ in (("t", torch.float64), ("r", torch.float32))}
    for bb in batches:
        cs = torch.tensor([p[1] for p in pairs if p[0] == bb])
        res = {}
        for tag, dtype in (("t", torch.float64), ("r", torch.float32)):
            leaf = dict(u=c(t["u"])[bb:bb + 1][:, cs], delta=c(t["delta"])[bb:bb + 1][:, cs], A=c(t["A"])[cs],
                        B=c(t["B"])[bb:bb + 1], C=c(t["C"])[bb:bb + 1], D=c(t["D"])[cs], z=c(t["z"])[bb:bb + 1][:, cs],
                        delta_bias=c(t["delta_bias"])[cs])
            leaf = {k: v.to(dtype).clone().requires_grad_(True) for k, v in leaf.items()}
            yo = OS6.selective_scan_ref(*[leaf[k] for k in keys], delta_softplus=True)
            (yo * c(gy)[bb:bb + 1][:, cs].to(dtype)).sum().backward()
            res[tag] = (yo.detach(), {k: v.grad for k, v in leaf.items()})
            for k in ("A", "D", "delta_bias"):
                acc[tag][k][cs] += leaf[k].grad
        assert_parity(f"s6 b{bb} out", c(y)[bb:bb + 1][:, cs], res["t"][0], res["r"][0])
        got = dict(u=c(t["u"].grad)[bb:bb + 1][:, cs], delta=c(t["delta"].grad)[bb:bb + 1][:, cs],
                   z=c(t["z"].grad)[bb:bb + 1][:, cs], B=c(t["B"].grad)[bb:bb + 1], C=c(t["C"].grad)[bb:bb + 1])
        for k, v in got.items():
            assert_parity(f"s6 b{bb} grad_{k}", v, res["t"][1][k], res["r"][1][k], atol=_gfloor(res["t"][1][k], l), rtol=1e-3)
    for k in ("A", "D", "delta_bias"):
        assert_parity(f"s6 grad_{k}", c(t[k].grad), acc["t"][k], acc["r"][k], atol=_gfloor(acc["t"][k], l), rtol=1e-3)
