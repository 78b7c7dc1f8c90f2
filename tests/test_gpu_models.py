"""The callers (AUSSM / Mamba blocks, SSMTS, SSMSequenceClassifier) on the CUDA operators against the same
modules evaluated on the CPU in float64 with the oracle's scans substituted for the operators."""
import pytest
import torch

import aussm_b200
from aussm_b200 import models, ops, s6
from aussm_b200.train import make_config, train_step
from oracle import unitary as OU
from oracle.s6 import selective_scan_ref
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu


def _oracle_interface(u, dt, x, x_bias, B, C, D, z, unitary=True, **kw):
    return OU.interface_unitary(u, dt, x, x_bias, B, C, D, z, recurrence=True)


def _reference_copy(model):
    """float64 CPU copy of the model whose scan calls go to the oracle"""
    import copy
    ref = copy.deepcopy(model).cpu().double()
    return ref


def _run_ref(ref, fn):
    saved = (ops.ssm_adaptive_interface, s6.selective_scan_fn)
    ops.ssm_adaptive_interface, s6.selective_scan_fn = _oracle_interface, selective_scan_ref
    try:
        return fn(ref)
    finally:
        ops.ssm_adaptive_interface, s6.selective_scan_fn = saved


def test_ssmts_hybrid_forward_backward_matches_oracle_model():
    torch.manual_seed(0)
    model = models.SSMTS(d_model=32, input_dim=5, output_dim=5, layers="a|m|a|m", d_state=8).cuda()
    ref = _reference_copy(model)
    x = torch.randn(3, 50, 5)
    y = torch.randn(3, 50, 5)
    out = model(x.cuda())
    torch.mean((out - y.cuda()) ** 2).backward()

    def go(m):
        o = m(x.double())
        torch.mean((o - y.double()) ** 2).backward()
        return o

    out64 = _run_ref(ref, go)
    assert_parity("output", out, out64, scaled_tol=2e-5)
    for (k, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        g, t = p.grad, q.grad
        if g.is_complex():
            g, t = torch.view_as_real(g), torch.view_as_real(t)
        assert_parity("grad " + k, g, t, atol=1e-5 * float(t.abs().max()) + 1e-9, rtol=1e-3, scaled_tol=2e-4)


def test_sequence_classifier_forward_matches_oracle_model():
    torch.manual_seed(1)
    model = models.SSMSequenceClassifier(d_model=16, vocab_size=11, output_dim=4, layers="a|a", d_state=4).cuda()
    ref = _reference_copy(model)
    ids = torch.randint(0, 11, (2, 70))
    out = model(ids.cuda())
    out64 = _run_ref(ref, lambda m: m(ids))
    assert_parity("logits", out, out64, scaled_tol=2e-5)
    lengths = torch.tensor([70, 33])
    out = model(ids.cuda(), lengths.cuda())
    out64 = _run_ref(ref, lambda m: m(ids, lengths))
    assert_parity("logits (lengths)", out, out64, scaled_tol=2e-5)


def test_reference_parameter_names():
    model = models.SSMTS(d_model=16, input_dim=3, output_dim=3, layers="a|m", d_state=4)
    names = set(dict(model.named_parameters()))
    for k in ["embedding.weight", "layers.0.mixer.xA_proj.weight", "layers.0.mixer.xA_proj.bias", "layers.0.mixer.B",
              "layers.0.mixer.C", "layers.0.mixer.D", "layers.0.mixer.dt_proj.bias", "layers.0.mixer.conv1d.weight",
              "layers.0.norm.weight", "layers.1.mixer.A_log", "layers.1.mixer.x_proj.weight", "norm_f.weight",
              "output.weight"]:
        assert k in names, k


@pytest.mark.parametrize("config", [3, 4])
def test_training_step_runs_and_reduces_the_loss(config):
    dev = torch.device("cuda", 0)
    model, batch, loss_fn, _, _, _ = make_config(config, dev, 0, 1, scale=0.05 if config == 3 else 0.002)
    opt = torch.optim.AdamW(model.parameters(), lr=2e-3)
    x, y = batch()
    x, y = x[:4], y[:4]
    first, _ = train_step(model, opt, x, y, loss_fn, 1, micro_batch=2)
    for _ in range(8):
        last, _ = train_step(model, opt, x, y, loss_fn, 1, micro_batch=2)
    assert last < first


def test_graphed_training_step_follows_the_eager_one():
    """The step captured into a CUDA graph and replayed does what the eager step does: same losses step by step (the
    Mamba layers' dB / dC use float atomics, so equality is up to rounding), and a new batch copied into the static
    inputs is used."""
    from aussm_b200.train import GraphedTrainStep
    dev = torch.device("cuda", 0)
    model_e, batch, loss_fn, _, _, _ = make_config(3, dev, 0, 1, scale=0.1)
    model_g, _, _, _, _, _ = make_config(3, dev, 0, 1, scale=0.1)          # same seed: same initial weights
    x, y = batch()
    x, y = x[:6], y[:6]
    x2 = torch.roll(x, 1, 0)
    opt_e = torch.optim.AdamW(model_e.parameters(), lr=2e-3)
    opt_g = torch.optim.AdamW(model_g.parameters(), lr=2e-3, capturable=True)
    for p, q in zip(model_e.parameters(), model_g.parameters()):
        assert torch.equal(p, q)
    start = {k: v.clone() for k, v in model_g.state_dict().items()}
    graphed = GraphedTrainStep(model_g, opt_g, x, y, loss_fn, micro_batch=3, warmup=2)
    # construction ran warm-up steps on the model: back to the start, optimizer state included
    model_g.load_state_dict(start)
    for st in opt_g.state.values():
        for v in st.values():
            if torch.is_tensor(v):
                v.zero_()
    for xs in (x, x, x2, x2):
        le, _ = train_step(model_e, opt_e, xs, y, loss_fn, 1, micro_batch=3)
        lg = float(graphed.step(xs, y))
        assert abs(le - lg) <= 1e-4 * max(1.0, abs(le)), (le, lg)
    for p, q in zip(model_e.parameters(), model_g.parameters()):
        assert torch.allclose(p, q, rtol=1e-3, atol=1e-4)
    assert aussm_b200.device_status() == 0


@pytest.mark.parametrize("shape", [(3, 50, 64, 128), (2, 7, 128, 36), (1, 1, 16, 8), (4, 33, 21, 128),
                                   (8, 2048, 64, 256)])
def test_split_linear_matches_float64(shape, monkeypatch):
    """SplitLinear == F.linear in float64 (forward and both gradients); sizes that are not multiples of 4 fall back;
    the last shape cuts the weight gradient's long contraction into slices."""
    import torch.nn.functional as F
    from aussm_b200 import linear
    from aussm_b200.linear import split_linear
    monkeypatch.setattr(linear, "MIN_FLOP", 0.0)
    b, l, d_in, d_out = shape
    gen = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(b, l, d_in, generator=gen)
    w = torch.randn(d_out, d_in, generator=gen) / d_in ** 0.5
    bias = torch.randn(d_out, generator=gen)
    gy = torch.randn(b, l, d_out, generator=gen)
    xs = [t.cuda().requires_grad_(True) for t in (x, w, bias)]
    y = split_linear(*xs)
    y.backward(gy.cuda())
    xd = [t.double().requires_grad_(True) for t in (x, w, bias)]
    yd = F.linear(*xd)
    yd.backward(gy.double())
    assert aussm_b200.device_status() == 0
    for name, got, want in [("y", y, yd)] + [(n, a.grad, c.grad) for n, a, c in zip(("x", "w", "b"), xs, xd)]:
        err = (got.detach().cpu().double() - want.detach()).abs().max().item()
        assert err <= 3e-6 * max(1.0, want.abs().max().item()), (name, err)
