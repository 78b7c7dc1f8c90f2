"""Host side of the B200 selective-scan operators.

This module mirrors the reference's operator front end,
extension-cpp/extension_cpp/ops.py: the same function names, argument order
and autograd contract, so that ``wavesAI.model.aussm.SSMauBlock`` can call it
unchanged (see ``install_as_extension_cpp``).  PyTorch only provides device
memory, streams and the autograd graph here; all arithmetic happens in
libaussm_b200.so.  There is no CPU or eager fallback: tensors must live on a
CUDA device and the library must be built.
"""
from __future__ import annotations

import os
import sys
import types
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from . import _lib

__all__ = ["ssm_adaptive_unitary", "ssm_adaptive_interface", "scan_unitary", "install_as_extension_cpp",
           "device_status"]

# ---------------------------------------------------------------------------
# Operator schemas: identical to the reference's TORCH_LIBRARY block
# (csrc/cuda/ssm_adaptive_unitary_forward.cu:283-286).
# ---------------------------------------------------------------------------
_FWD_SCHEMA = ("ssm_adaptive_unitary(Tensor u,Tensor dt,Tensor x, Tensor x_bias, Tensor B_r, Tensor B_theta, "
               "Tensor C_r, Tensor C_theta, Tensor D, Tensor z, Tensor prev_hid_real, "
               "Tensor prev_hidden_state_imag) -> (Tensor, Tensor, Tensor)")
_BWD_SCHEMA = ("ssm_adaptive_backward_unitary(Tensor grad_y,Tensor grad_next_hid_real,Tensor grad_next_hid_imag,"
               "Tensor u,Tensor dt,Tensor x,Tensor x_bias,Tensor B_r,Tensor B_theta,Tensor C_r,Tensor C_theta,"
               "Tensor D,Tensor z, Tensor prev_hid_real, Tensor prev_hid_imag) -> (Tensor, Tensor, Tensor, Tensor, "
               "Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")

_library = torch.library.Library("extension_cpp", "DEF")
_library.define(_FWD_SCHEMA)
_library.define(_BWD_SCHEMA)


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(t: Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _f32c(name: str, t: Tensor, shape=None) -> Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU implementation of this operator)")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise RuntimeError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
    return t.contiguous()


def _workspace(nbytes: int, device) -> Tensor:
    # torch's caching allocator hands out 512-byte aligned blocks
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def device_status(device=None) -> int:
    """Synchronise the current stream of `device` and return (and clear) the status word of that device's kernels.

    0 = every kernel ran to completion; 1 = a kernel gave up on a bounded wait (its outputs are then invalid).
    The operators do not poll this word themselves unless ``check_device_status`` is set, because reading it
    synchronises the stream."""
    with torch.cuda.device(device):            # the word is per device: read the one that owns the stream
        stream = torch.cuda.current_stream().cuda_stream
        return int(_lib.load().aussm_b200_device_status(stream))


# Opt-in polling of the device status word: when true (or when the environment variable
# AUSSM_B200_CHECK_STATUS=1 is set at import), every drop-in operator call and every training step synchronises
# its stream once and raises if a kernel reported a timed-out wait, instead of handing on invalid values.
check_device_status = os.environ.get("AUSSM_B200_CHECK_STATUS", "0") == "1"


def _poll_status(what: str, device) -> None:
    if check_device_status and device_status(device) != 0:
        raise RuntimeError(f"{what}: a kernel gave up on a bounded wait (device status word set); outputs are invalid")


# ---------------------------------------------------------------------------
# Drop-in operator pair
# ---------------------------------------------------------------------------
def _check_op_inputs(u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im):
    if u.dim() != 3:
        raise RuntimeError(f"u must be (batch, d, length), got {tuple(u.shape)}")
    b, d, l = u.shape
    if x.dim() != 3 or x.shape[0] != d or x.shape[2] != d:
        raise RuntimeError(f"x must be (d, n, d) with d={d}, got {tuple(x.shape)}")
    n = x.shape[1]
    u = _f32c("u", u)
    return (b, d, n, l,
            u, _f32c("dt", dt, (b, d, l)), _f32c("x", x, (d, n, d)), _f32c("x_bias", x_bias, (d, n)),
            _f32c("B_r", B_r, (n,)), _f32c("B_theta", B_theta, (n,)), _f32c("C_r", C_r, (n,)),
            _f32c("C_theta", C_theta, (n,)), _f32c("D", D, (d,)), _f32c("z", z, (b, d, l)),
            _f32c("prev_hid_real", h_re, (b, d, n)), _f32c("prev_hid_imag", h_im, (b, d, n)))


def _unitary_forward(u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im):
    (b, d, n, l, u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im) = _check_op_inputs(
        u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im)
    lib = _lib.load()
    y = torch.empty_like(u)
    o_re = torch.empty_like(h_re)
    o_im = torch.empty_like(h_im)
    if l == 0 or b == 0:
        o_re.copy_(h_re)
        o_im.copy_(h_im)
        return y, o_re, o_im
    with torch.cuda.device(u.device):
        nbytes = lib.aussm_b200_unitary_workspace_bytes(b, d, n, l)
        ws = _workspace(nbytes, u.device)
        rc = lib.aussm_b200_unitary_fwd(
            _ptr(u), _ptr(dt), _ptr(x), _ptr(x_bias), _ptr(B_r), _ptr(B_theta), _ptr(C_r), _ptr(C_theta), _ptr(D),
            _ptr(z), _ptr(h_re), _ptr(h_im), _ptr(y), _ptr(o_re), _ptr(o_im), b, d, n, l, _ptr(ws), ws.numel(),
            _stream(u))
    _lib.check(rc, "ssm_adaptive_unitary")
    _poll_status("ssm_adaptive_unitary", u.device)
    return y, o_re, o_im


def _unitary_backward(grad_y, g_re, g_im, u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im,
                      final_state=None, keep=None):
    (b, d, n, l, u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im) = _check_op_inputs(
        u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im)
    lib = _lib.load()
    grad_y = _f32c("grad_y", grad_y, (b, d, l))
    g_re = None if g_re is None else _f32c("grad_next_hid_real", g_re, (b, d, n))
    g_im = None if g_im is None else _f32c("grad_next_hid_imag", g_im, (b, d, n))
    if (g_re is None) != (g_im is None):
        zero = torch.zeros_like(h_re)
        g_re = zero if g_re is None else g_re
        g_im = zero if g_im is None else g_im
    f_re = f_im = None
    if final_state is not None:
        f_re = _f32c("next_hid_real", final_state[0], (b, d, n))
        f_im = _f32c("next_hid_imag", final_state[1], (b, d, n))
    du, ddt, dz = torch.empty_like(u), torch.empty_like(u), torch.empty_like(u)
    dx, dxb = torch.empty_like(x), torch.empty_like(x_bias)
    dBr, dBt, dCr, dCt = (torch.empty_like(B_r) for _ in range(4))
    dD = torch.empty_like(D)
    dh_re, dh_im = torch.empty_like(h_re), torch.empty_like(h_im)
    if l == 0 or b == 0:
        for t in (du, ddt, dz, dx, dxb, dBr, dBt, dCr, dCt, dD):
            t.zero_()
        dh_re.copy_(g_re if g_re is not None else torch.zeros_like(h_re))
        dh_im.copy_(g_im if g_im is not None else torch.zeros_like(h_im))
        return du, ddt, dx, dxb, dBr, dBt, dCr, dCt, dD, dz, dh_re, dh_im
    with torch.cuda.device(u.device):
        nbytes = lib.aussm_b200_unitary_workspace_bytes(b, d, n, l)
        ws = _workspace(nbytes, u.device)
        args = (_ptr(grad_y), _ptr(g_re), _ptr(g_im), _ptr(u), _ptr(dt), _ptr(x), _ptr(x_bias), _ptr(B_r),
                _ptr(B_theta), _ptr(C_r), _ptr(C_theta), _ptr(D), _ptr(z), _ptr(h_re), _ptr(h_im), _ptr(f_re),
                _ptr(f_im), _ptr(du), _ptr(ddt), _ptr(dx), _ptr(dxb), _ptr(dBr), _ptr(dBt), _ptr(dCr), _ptr(dCt),
                _ptr(dD), _ptr(dz), _ptr(dh_re), _ptr(dh_im), b, d, n, l, _ptr(ws), ws.numel())
        if keep is not None:
            rc = lib.aussm_b200_unitary_bwd_kept(*args, _ptr(keep), keep.numel(), _stream(u))
        else:
            rc = lib.aussm_b200_unitary_bwd(*args, _stream(u))
    _lib.check(rc, "ssm_adaptive_backward_unitary")
    _poll_status("ssm_adaptive_backward_unitary", u.device)
    return du, ddt, dx, dxb, dBr, dBt, dCr, dCt, dD, dz, dh_re, dh_im


_library.impl("ssm_adaptive_unitary", _unitary_forward, "CUDA")
_library.impl("ssm_adaptive_backward_unitary", _unitary_backward, "CUDA")


def _no_cpu(*args, **kwargs):
    raise RuntimeError("extension_cpp::ssm_adaptive_unitary has no CPU implementation in aussm_b200; "
                       "move the tensors to a CUDA device")


_library.impl("ssm_adaptive_unitary", _no_cpu, "CPU")
_library.impl("ssm_adaptive_backward_unitary", _no_cpu, "CPU")


@torch.library.register_fake("extension_cpp::ssm_adaptive_unitary")
def _fake_forward(u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, prev_hid_real, prev_hidden_state_imag):
    # the reference's fake implementation (ops.py:156-165) has the wrong arity; this one matches the schema
    return torch.empty_like(u), torch.empty_like(prev_hid_real), torch.empty_like(prev_hidden_state_imag)


@torch.library.register_fake("extension_cpp::ssm_adaptive_backward_unitary")
def _fake_backward(grad_y, g_re, g_im, u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im):
    return tuple(torch.empty_like(t) for t in (u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im))


# Whether a differentiable call keeps its phase tensor (4*b*d*n*l bytes) for the backward pass, which then
# skips one of the four projection GEMMs: True, False, or "auto" = when it takes at most a quarter of the
# device memory that is free at the time of the call.  Results are bit-identical either way.
keep_phases = "auto"


def _want_keep(inputs, b, d, n, l) -> int:
    """Size of the phase buffer to keep for this call, or 0 for the recomputing path."""
    if keep_phases is False or not torch.is_grad_enabled() or not any(t.requires_grad for t in inputs):
        return 0
    if b == 0 or l == 0:
        return 0
    nbytes = _lib.load().aussm_b200_unitary_keep_bytes(b, d, n, l)
    if keep_phases is True:
        return nbytes
    free, _total = torch.cuda.mem_get_info(inputs[0].device)
    return nbytes if nbytes <= free // 4 else 0


class _UnitaryKeep(torch.autograd.Function):
    """extension_cpp::ssm_adaptive_unitary with the phases kept for the backward pass."""

    @staticmethod
    def forward(ctx, keep_bytes, *inputs):
        (b, d, n, l, u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im) = _check_op_inputs(*inputs)
        lib = _lib.load()
        y, o_re, o_im = torch.empty_like(u), torch.empty_like(h_re), torch.empty_like(h_im)
        keep = torch.empty(keep_bytes, dtype=torch.uint8, device=u.device)
        with torch.cuda.device(u.device):
            ws = _workspace(lib.aussm_b200_unitary_workspace_bytes(b, d, n, l), u.device)
            rc = lib.aussm_b200_unitary_fwd_keep(
                _ptr(u), _ptr(dt), _ptr(x), _ptr(x_bias), _ptr(B_r), _ptr(B_theta), _ptr(C_r), _ptr(C_theta),
                _ptr(D), _ptr(z), _ptr(h_re), _ptr(h_im), _ptr(y), _ptr(o_re), _ptr(o_im), b, d, n, l, _ptr(ws),
                ws.numel(), _ptr(keep), keep.numel(), _stream(u))
        _lib.check(rc, "ssm_adaptive_unitary (phases kept)")
        _poll_status("ssm_adaptive_unitary (phases kept)", u.device)
        ctx.save_for_backward(u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h_re, h_im, o_re, o_im)
        ctx.keep = keep
        return y, o_re, o_im

    @staticmethod
    def backward(ctx, grad_y, g_re, g_im):
        saved = ctx.saved_tensors
        inputs, f_re, f_im = saved[:12], saved[12], saved[13]
        if grad_y is None:
            grad_y = torch.zeros_like(inputs[0])
        keep, ctx.keep = ctx.keep, None        # the backward call overwrites the phases: usable once
        return (None,) + tuple(_unitary_backward(grad_y, g_re, g_im, *inputs, final_state=(f_re, f_im), keep=keep))


def ssm_adaptive_unitary(u: Tensor, dt: Tensor, x: Tensor, x_bias: Tensor, B_r: Tensor, B_theta: Tensor,
                         C_r: Tensor, C_theta: Tensor, D: Tensor, z: Tensor, prev_hidden_state_real: Tensor,
                         prev_hidden_state_imag: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """The operator call of the reference (ops.py:97-105): returns (y, next_hid_real, next_hid_imag)."""
    inputs = (u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, prev_hidden_state_real, prev_hidden_state_imag)
    if u.is_cuda and u.dim() == 3 and x.dim() == 3:
        keep_bytes = _want_keep(inputs, u.shape[0], u.shape[1], x.shape[1], u.shape[2])
        if keep_bytes:
            return _UnitaryKeep.apply(keep_bytes, *inputs)
    return torch.ops.extension_cpp.ssm_adaptive_unitary.default(*inputs)


def _setup_context(ctx, inputs, output):
    # The reference saves the 12 inputs only (ops.py:148-151) and its backward
    # kernel recomputes the states.  Saving the two small final-state outputs as
    # well lets the backward pass start from them (the recurrence is reversible)
    # instead of re-running the forward sweep.
    ctx.save_for_backward(*inputs, output[1], output[2])


def _backward(ctx, grad_y, grad_next_hid_real, grad_next_hid_imag):
    saved = ctx.saved_tensors
    inputs, f_re, f_im = saved[:12], saved[12], saved[13]
    if grad_y is None:
        grad_y = torch.zeros_like(inputs[0])
    try:
        return _unitary_backward(grad_y, grad_next_hid_real, grad_next_hid_imag, *inputs, final_state=(f_re, f_im))
    except RuntimeError:
        # same diagnostic as the reference (ops.py:133-143)
        names = ["u", "dt", "x", "x_bias", "B_r", "B_theta", "C_r", "C_theta", "D", "z"]
        shapes = {k: tuple(t.shape) for k, t in zip(names, inputs)}
        shapes["grad_y"] = tuple(grad_y.shape)
        print(f"Runtime Error for {shapes}")
        raise


torch.library.register_autograd("extension_cpp::ssm_adaptive_unitary", _backward, setup_context=_setup_context)


def pad_to_multiple_of(tensor: Tensor, multiple_of: int) -> Tensor:
    """Zero-pad the last axis up to a multiple (reference: ops.py:21-25)."""
    pad = (-tensor.shape[-1]) % multiple_of
    return F.pad(tensor, (0, pad)) if pad else tensor


def ssm_adaptive_interface(u: Tensor, dt: Tensor, x: Tensor, x_bias: Tensor, B: Tensor, C: Tensor, D: Tensor,
                           z: Tensor, unitary=True, preal=False, max_parallel_length=2048, **kwargs) -> Tensor:
    """Front end with the reference's signature and semantics (ops.py:28-93).

    ``u, dt, z`` are ``(b, d, l)``, ``x`` is ``(d, n, d)``, ``x_bias`` ``(d, n)``, ``B, C`` complex ``(n,)``
    (radius = softplus(real part), angle = imaginary part), ``D`` ``(d,)``.  Unknown keyword arguments
    are ignored, as in the reference.  ``max_parallel_length`` exists because the reference kernels
    handle at most 2048 steps per launch; the kernels here have no such limit, so the default (and any
    larger value) runs the whole sequence in one operator call, while a smaller value is honoured and
    splits the sequence into chunks that hand the complex hidden state on (same result).
    """
    assert not (unitary and preal), "Both unitary and preal cannot be used at the same time"
    if not unitary:
        raise NotImplementedError("other kernels not implemented")
    initial_length = u.shape[-1]
    b, d, _ = u.shape
    n = x.shape[1]
    u = pad_to_multiple_of(u, 16).contiguous()
    dt = pad_to_multiple_of(dt, 16).contiguous()
    z = pad_to_multiple_of(z, 16).contiguous()
    l = u.shape[-1]
    B_r = F.softplus(B.real).contiguous()
    B_theta = B.imag.contiguous()
    C_r = F.softplus(C.real).contiguous()
    C_theta = C.imag.contiguous()
    h_re = torch.zeros((b, d, n), device=u.device, dtype=torch.float32)
    h_im = torch.zeros((b, d, n), device=u.device, dtype=torch.float32)
    chunk = l if max_parallel_length is None or max_parallel_length >= 2048 else int(max_parallel_length)
    if chunk >= l:
        out, _, _ = ssm_adaptive_unitary(u, dt, x.contiguous(), x_bias.contiguous(), B_r, B_theta, C_r, C_theta,
                                         D.contiguous(), z, h_re, h_im)
    else:
        pieces = []
        for s in range(0, l, chunk):
            e = min(s + chunk, l)
            y_c, h_re, h_im = ssm_adaptive_unitary(u[:, :, s:e].contiguous(), dt[:, :, s:e].contiguous(),
                                                   x.contiguous(), x_bias.contiguous(), B_r, B_theta, C_r, C_theta,
                                                   D.contiguous(), z[:, :, s:e].contiguous(), h_re, h_im)
            pieces.append(y_c)
        out = torch.cat(pieces, dim=-1)
    return out[:, :, :initial_length]


# ---------------------------------------------------------------------------
# Scan core (phase tensor given): the memory-bound part, exposed for
# measurement and for callers that produce theta themselves.
# ---------------------------------------------------------------------------
class _ScanUnitary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, theta, u, dt, z, B_r, B_theta, C_r, C_theta, D, h0_re, h0_im):
        b, d, n, l = theta.shape
        theta = _f32c("theta", theta)
        u, dt, z = _f32c("u", u, (b, d, l)), _f32c("dt", dt, (b, d, l)), _f32c("z", z, (b, d, l))
        B_r, B_theta = _f32c("B_r", B_r, (n,)), _f32c("B_theta", B_theta, (n,))
        C_r, C_theta = _f32c("C_r", C_r, (n,)), _f32c("C_theta", C_theta, (n,))
        D = _f32c("D", D, (d,))
        h0_re = None if h0_re is None else _f32c("h0_re", h0_re, (b, d, n))
        h0_im = None if h0_im is None else _f32c("h0_im", h0_im, (b, d, n))
        y = torch.empty_like(u)
        h_re = torch.empty((b, d, n), device=u.device, dtype=torch.float32)
        h_im = torch.empty_like(h_re)
        lib = _lib.load()
        with torch.cuda.device(u.device):
            # the workspace is non-empty only when the launch is cut into time segments (few channels)
            nbytes = lib.aussm_b200_scan_unitary_fwd_workspace_bytes(b, d, n, l)
            ws = _workspace(nbytes, u.device) if nbytes else None
            rc = lib.aussm_b200_scan_unitary_fwd_ws(
                _ptr(theta), _ptr(u), _ptr(dt), _ptr(z), _ptr(B_r), _ptr(B_theta), _ptr(C_r), _ptr(C_theta), _ptr(D),
                _ptr(h0_re), _ptr(h0_im), _ptr(y), _ptr(h_re), _ptr(h_im), b, d, n, l, _ptr(ws),
                0 if ws is None else ws.numel(), _stream(u))
        _lib.check(rc, "scan_unitary forward")
        ctx.save_for_backward(theta, u, dt, z, B_r, B_theta, C_r, C_theta, D, h_re, h_im)
        ctx.has_h0 = h0_re is not None
        return y, h_re, h_im

    @staticmethod
    def backward(ctx, gy, g_re, g_im):
        theta, u, dt, z, B_r, B_theta, C_r, C_theta, D, h_re, h_im = ctx.saved_tensors
        b, d, n, l = theta.shape
        lib = _lib.load()
        gy = torch.zeros_like(u) if gy is None else _f32c("grad_y", gy, (b, d, l))
        if (g_re is None) != (g_im is None):
            zero = torch.zeros_like(h_re)
            g_re = zero if g_re is None else g_re
            g_im = zero if g_im is None else g_im
        g_re = None if g_re is None else _f32c("gh_re", g_re, (b, d, n))
        g_im = None if g_im is None else _f32c("gh_im", g_im, (b, d, n))
        dtheta = torch.empty_like(theta)
        du, ddt, dz = torch.empty_like(u), torch.empty_like(u), torch.empty_like(u)
        dBr, dBt, dCr, dCt = (torch.empty_like(B_r) for _ in range(4))
        dD = torch.empty_like(D)
        dh_re, dh_im = torch.empty_like(h_re), torch.empty_like(h_im)
        with torch.cuda.device(u.device):
            ws = _workspace(lib.aussm_b200_scan_unitary_bwd_workspace_bytes(b, d, n, l), u.device)
            rc = lib.aussm_b200_scan_unitary_bwd(
                _ptr(gy), _ptr(g_re), _ptr(g_im), _ptr(theta), _ptr(u), _ptr(dt), _ptr(z), _ptr(B_r), _ptr(B_theta),
                _ptr(C_r), _ptr(C_theta), _ptr(D), _ptr(h_re), _ptr(h_im), _ptr(dtheta), _ptr(du), _ptr(ddt),
                _ptr(dz), _ptr(dBr), _ptr(dBt), _ptr(dCr), _ptr(dCt), _ptr(dD), _ptr(dh_re), _ptr(dh_im), b, d, n,
                l, _ptr(ws), ws.numel(), _stream(u))
        _lib.check(rc, "scan_unitary backward")
        if not ctx.has_h0:
            dh_re = dh_im = None
        return dtheta, du, ddt, dz, dBr, dBt, dCr, dCt, dD, dh_re, dh_im


def scan_unitary(theta: Tensor, u: Tensor, dt: Tensor, z: Tensor, B_r: Tensor, B_theta: Tensor, C_r: Tensor,
                 C_theta: Tensor, D: Tensor, h0_re: Optional[Tensor] = None,
                 h0_im: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """Unitary scan on a given phase tensor ``theta`` of shape ``(b, d, n, l)``.

    Returns ``(y, h_re, h_im)``; differentiable in every argument.
    """
    return _ScanUnitary.apply(theta, u, dt, z, B_r, B_theta, C_r, C_theta, D, h0_re, h0_im)


# ---------------------------------------------------------------------------
# Drop-in registration under the reference's package name
# ---------------------------------------------------------------------------
def install_as_extension_cpp() -> types.ModuleType:
    """Make ``import extension_cpp`` resolve to this implementation.

    ``wavesAI.model.aussm`` does ``import extension_cpp`` and calls
    ``extension_cpp.ops.ssm_adaptive_interface`` (aussm.py:836-840); after this call it gets the
    functions of this module.  Refuses to shadow a real ``extension_cpp`` that is already imported.
    """
    existing = sys.modules.get("extension_cpp")
    if existing is not None and not getattr(existing, "_aussm_b200_shim", False):
        raise RuntimeError("a different extension_cpp package is already imported")
    pkg = types.ModuleType("extension_cpp")
    pkg._aussm_b200_shim = True
    pkg.ops = sys.modules[__name__]
    pkg.__path__ = []
    sys.modules["extension_cpp"] = pkg
    sys.modules["extension_cpp.ops"] = sys.modules[__name__]
    return pkg
