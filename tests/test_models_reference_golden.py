"""aussm_b200.models against the REFERENCE's own model classes.

tests/golden/model_*.npz hold a state_dict, an input, and the output and
parameter gradients that the reference's ``ai-modules/wavesAI/model/aussm.py``
classes gave for them on the CPU (made by tests/golden/make_models_golden.py).
The state_dict is loaded into this package's restatement of the class:

* on the CPU in float64, with the oracle's scans substituted for the CUDA
  operators: pins the module glue (layer order, the doubled dt_proj bias, the
  ``(n d1) d`` view of xA_proj, silu before the Mamba scan, pooling modes)
  to 1e-9;
* on the GPU in float32 through the CUDA operators, to the parity tolerance.
"""
import ast

import numpy as np
import pytest
import torch

from aussm_b200 import models, ops, s6
from oracle import unitary as OU
from oracle.s6 import selective_scan_ref
from tests.helpers import GOLDEN, assert_parity

import os

CASES = {
    "model_ssmts_aa": models.SSMTS,
    "model_classifier_aa": models.SSMSequenceClassifier,
    "model_classifier_aa_lengths": models.SSMSequenceClassifier,
    "model_classifier_last": models.SSMSequenceClassifier,
    "model_ssmts_am_glue": models.SSMTS,
}


def _load(name):
    blob = np.load(os.path.join(GOLDEN, name + ".npz"))
    ctor = ast.literal_eval(str(blob["ctor"]))
    state = {k[len("state."):]: torch.from_numpy(blob[k]) for k in blob.files if k.startswith("state.")}
    grads = {k[len("grad64."):]: torch.from_numpy(blob[k]) for k in blob.files if k.startswith("grad64.")}
    inputs = [torch.from_numpy(blob[k]) for k in sorted(f for f in blob.files if f.startswith("input"))]
    return ctor, state, inputs, torch.from_numpy(blob["out32"]), torch.from_numpy(blob["out64"]), grads


def _oracle_interface(u, dt, x, x_bias, B, C, D, z, unitary=True, **kw):
    return OU.interface_unitary(u, dt, x, x_bias, B, C, D, z, recurrence=True)


def _real(t):
    return torch.view_as_real(t) if t.is_complex() else t


@pytest.mark.parametrize("name", list(CASES))
def test_module_glue_matches_reference_classes_on_cpu(name):
    ctor, state, inputs, _out32, out64, grads = _load(name)
    model = CASES[name](**ctor)
    missing = model.load_state_dict(state, strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    model = model.double()
    for p in model.parameters():
        if p.is_complex():             # Module.double() leaves the complex parameters alone
            p.data = p.data.to(torch.complex128)
    saved = (ops.ssm_adaptive_interface, s6.selective_scan_fn)
    ops.ssm_adaptive_interface, s6.selective_scan_fn = _oracle_interface, selective_scan_ref
    try:
        out = model(*[a.double() if a.is_floating_point() else a for a in inputs])
        (out ** 2).mean().backward()
    finally:
        ops.ssm_adaptive_interface, s6.selective_scan_fn = saved
    torch.testing.assert_close(out.reshape(out64.shape), out64, rtol=1e-9, atol=1e-10)
    got = dict(model.named_parameters())
    assert set(got) == set(grads)
    for k, g in grads.items():
        torch.testing.assert_close(_real(got[k].grad), _real(g), rtol=1e-6, atol=1e-10, msg=lambda m, k=k: f"{k}: {m}")


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_cuda_models_match_reference_classes(name):
    ctor, state, inputs, out32, out64, grads = _load(name)
    model = CASES[name](**ctor)
    model.load_state_dict(state, strict=True)
    model = model.cuda()
    out = model(*[a.cuda() for a in inputs])
    (out ** 2).mean().backward()
    import aussm_b200
    assert aussm_b200.device_status() == 0
    assert_parity(f"{name} output", out.reshape(out64.shape), out64, out32)
    for k, p in model.named_parameters():
        t = _real(grads[k])
        assert_parity(f"{name} grad {k}", _real(p.grad), t, atol=1e-5 * float(t.abs().max()) + 1e-12, rtol=1e-3,
                      scaled_tol=2e-4)
