"""Generate golden vectors of the reference's MODEL classes (its own ``aussm.py``),
so that ``aussm_b200.models`` can be checked against the originals without a
checkout:

    python tests/golden/make_models_golden.py /path/to/AUSSM

``ai-modules/wavesAI/model/aussm.py`` is loaded by path, on the CPU.  What it
imports and this machine lacks is stubbed: plotting / debugging modules
(matplotlib, icecream: unused by the classes), ``extension_cpp`` (a package
object whose ``ops`` is the reference's own ``extension_cpp/ops.py`` loaded by
path after its two operator schemas have been defined - see make_golden.py),
and ``mamba_ssm`` (third-party, absent from the reference tree).  The AUSSM
blocks run the reference's CPU path, ``cuda=False`` (aussm.py:841-843:
``reference_ssm_adaptive_unitary_optimized_polar``), with ``torch.compile``
turned into the identity so that the eager function runs.  Stored per case:
the ``state_dict``, the input, the output in float32 and float64, and the
float64 gradient of ``mean(out^2)`` with respect to every parameter.

The hybrid case ('a|m') needs ``mamba_ssm``'s ``selective_scan_fn``; there the
stub is this repository's own restatement of the S6 recurrence
(oracle/s6.py), so that case pins the Mamba block's glue code (the order of
silu, convolution, dt_proj and its doubled bias, aussm.py:771-805) to the
reference class but NOT the scan arithmetic, which stays unpinned.
"""
from __future__ import annotations

import contextlib
import importlib.util
import io
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from make_golden import load_reference_ops  # noqa: E402
from oracle.s6 import selective_scan_ref  # noqa: E402


def load_reference_models(root: str):
    ref_ops = load_reference_ops(root)
    pkg = types.ModuleType("extension_cpp")
    pkg.ops = ref_ops
    sys.modules["extension_cpp"] = pkg
    sys.modules["extension_cpp.ops"] = ref_ops
    for name in ("matplotlib", "matplotlib.pyplot", "icecream", "mamba_ssm", "mamba_ssm.ops",
                 "mamba_ssm.ops.selective_scan_interface"):
        if name not in sys.modules:
            sys.modules[name] = types.ModuleType(name)
    sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    sys.modules["icecream"].ic = lambda *a, **k: None
    sys.modules["mamba_ssm.ops.selective_scan_interface"].selective_scan_fn = selective_scan_ref
    torch.compile = lambda fn=None, *a, **k: fn            # the cuda=False path wraps the oracle in torch.compile
    path = os.path.join(root, "ai-modules", "wavesAI", "model", "aussm.py")
    spec = importlib.util.spec_from_file_location("_reference_aussm", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["_reference_aussm"] = mod
    with contextlib.redirect_stdout(io.StringIO()):
        spec.loader.exec_module(mod)
    return mod, ref_ops


def _force_cpu_path(model, ref_ops):
    """SSMSequenceClassifier has no ssmau_cuda switch: give its AUSSM blocks the function their cuda=False
    branch would have chosen (aussm.py:841-843)."""
    for m in model.modules():
        if hasattr(m, "optimized_SSMa_function"):
            m.optimized_SSMa_function = ref_ops.reference_ssm_adaptive_unitary_optimized_polar


def _run(model, inputs, dtype):
    m = model.double() if dtype == torch.float64 else model.float()
    for p in m.parameters():
        p.grad = None
        if p.is_complex():             # Module.double() leaves complex parameters (B, C of the AUSSM blocks) alone
            p.data = p.data.to(torch.complex128 if dtype == torch.float64 else torch.complex64)
    args = [a.to(dtype) if a.is_floating_point() else a for a in inputs]
    with contextlib.redirect_stdout(io.StringIO()):
        out = m(*args)
    (out ** 2).mean().backward()
    grads = {k: p.grad.detach().clone() for k, p in m.named_parameters()}
    return out.detach().clone(), grads


def save_case(name, model, inputs, ref_ops, ctor):
    _force_cpu_path(model, ref_ops)
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}       # float32 originals
    out32, _ = _run(model, inputs, torch.float32)
    out64, g64 = _run(model, inputs, torch.float64)
    blob = {"ctor": np.array(repr(ctor))}
    for i, a in enumerate(inputs):
        blob[f"input{i}"] = a.numpy()
    for k, v in state.items():
        blob["state." + k] = v.numpy()
    blob["out32"] = out32.numpy()
    blob["out64"] = out64.numpy()
    for k, v in g64.items():
        blob["grad64." + k] = v.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
    print(name, tuple(out64.shape), f"{sum(v.numel() for v in state.values())} parameters")


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AUSSM_REFERENCE_ROOT", "")
    if not root or not os.path.isdir(root):
        raise SystemExit("usage: make_models_golden.py <path to an AUSSM checkout>")
    ref, ref_ops = load_reference_models(root)
    quiet = contextlib.redirect_stdout(io.StringIO())

    torch.manual_seed(101)
    ctor = dict(d_model=16, input_dim=5, output_dim=3, layers="a|a", d_state=4)
    with quiet:
        m = ref.SSMTS(**ctor, ssmau_cuda=False, verbose=False)
    save_case("model_ssmts_aa", m, [torch.randn(2, 24, 5)], ref_ops, ctor)

    torch.manual_seed(102)
    ctor = dict(d_model=16, vocab_size=11, output_dim=4, layers="a|a", d_state=4)
    with quiet:
        m = ref.SSMSequenceClassifier(**ctor, verbose=False)
    save_case("model_classifier_aa", m, [torch.randint(0, 11, (3, 20))], ref_ops, ctor)
    save_case("model_classifier_aa_lengths", m, [torch.randint(0, 11, (3, 20)), torch.tensor([20, 7, 13])], ref_ops,
              ctor)

    torch.manual_seed(103)
    ctor = dict(d_model=16, vocab_size=11, output_dim=4, layers="a", d_state=4, mode="last")
    with quiet:
        m = ref.SSMSequenceClassifier(**ctor, verbose=False)
    save_case("model_classifier_last", m, [torch.randint(0, 11, (3, 20))], ref_ops, ctor)

    torch.manual_seed(104)
    ctor = dict(d_model=16, input_dim=5, output_dim=5, layers="a|m", d_state=8)
    with quiet:
        m = ref.SSMTS(**ctor, ssmau_cuda=False, verbose=False)
    save_case("model_ssmts_am_glue", m, [torch.randn(2, 20, 5)], ref_ops, ctor)


if __name__ == "__main__":
    main()
