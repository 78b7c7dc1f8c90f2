"""The AUSSM block's stages around the scan operator, in the scan's own (batch, channel, time) layout.

The reference's ``SSMauBlock`` (ai-modules/wavesAI/model/aussm.py:849-902) works token-major, ``(b, l, d)``,
and transposes to ``(b, d, l)`` and back around its convolution and around the operator (four transposing
copies per call, :858-864 and :888-897), applies the convolution through ``nn.Conv1d`` with padding and a
slice, and builds the step size with separate bias-add and softplus passes (:878-880).  Here every stage
produces its result directly in ``(b, d, l)``:

* ``project_tokens`` / ``project_channels`` / ``project_back``: the block's linear layers as matrix products
  whose output (or input) is channel-major, so no transposing copy exists.  Large products run on the
  library's split GEMM (float32-accurate, tcgen05), small ones on ``torch.matmul`` over views;
* ``causal_conv_bias``: depthwise causal convolution + bias, one pass (``aussm_b200_conv_pre_fwd/_bwd``);
* ``softplus_bias``: ``softplus(pre + scale * bias)``, one pass, in place (``aussm_b200_softplus_bias_fwd/_bwd``).

All functions are differentiable.  CUDA float32 tensors only.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _lib
from .ops import _f32c, _ptr, _stream, _workspace
from .variants import _gemm

__all__ = ["causal_conv_bias", "softplus_bias", "project_tokens", "project_channels", "project_back"]

# Below this many floating-point operations a product runs on torch.matmul (over views: still no copies); the
# split GEMM spends two passes over each operand on its FP16 parts before the product starts.
MIN_FLOP = 2.0e10


# ---------------------------------------------------------------------------
# element-wise stages
# ---------------------------------------------------------------------------
class _CausalConvBias(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xs, weight, bias):
        b, d, l = xs.shape
        k = weight.shape[-1]
        lib = _lib.load()
        u = torch.empty_like(xs)
        w2 = weight.reshape(d, k).contiguous()
        with torch.cuda.device(xs.device):
            rc = lib.aussm_b200_conv_pre_fwd(_ptr(xs), _ptr(w2), _ptr(bias), _ptr(u), b, d, l, k, _stream(xs))
        _lib.check(rc, "causal_conv_bias")
        ctx.save_for_backward(xs, w2)
        ctx.has_bias = bias is not None
        ctx.wshape = weight.shape
        return u

    @staticmethod
    def backward(ctx, du):
        xs, w2 = ctx.saved_tensors
        b, d, l = xs.shape
        k = w2.shape[1]
        lib = _lib.load()
        du = du.contiguous()
        dxs = torch.empty_like(xs)
        dw = torch.empty_like(w2)
        dbias = torch.empty(d, device=xs.device, dtype=torch.float32) if ctx.has_bias else None
        with torch.cuda.device(xs.device):
            ws = _workspace(lib.aussm_b200_conv_pre_bwd_workspace_bytes(b, d), xs.device)
            rc = lib.aussm_b200_conv_pre_bwd(_ptr(du), _ptr(xs), _ptr(w2), _ptr(dxs), _ptr(dw), _ptr(dbias), b, d, l, k,
                                             _ptr(ws), ws.numel(), _stream(xs))
        _lib.check(rc, "causal_conv_bias backward")
        return dxs, dw.view(ctx.wshape), dbias


def causal_conv_bias(xs: Tensor, weight: Tensor, bias: Tensor = None) -> Tensor:
    """``conv1d(xs, weight, bias, padding=k-1, groups=d)[..., :l]`` for ``xs`` (b, d, l) and ``weight``
    (d, 1, k), k <= 4: the block's causal depthwise convolution (aussm.py:858-864) in one pass."""
    b, d, l = xs.shape
    return _CausalConvBias.apply(_f32c("xs", xs, (b, d, l)), _f32c("conv weight", weight),
                                 None if bias is None else _f32c("conv bias", bias, (d,)))


class _SoftplusBias(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pre, bias, scale):
        b, d, l = pre.shape
        lib = _lib.load()
        dt = torch.empty_like(pre)
        with torch.cuda.device(pre.device):
            rc = lib.aussm_b200_softplus_bias_fwd(_ptr(pre), _ptr(bias), float(scale), _ptr(dt), b, d, l, _stream(pre))
        _lib.check(rc, "softplus_bias")
        ctx.save_for_backward(dt)
        ctx.scale = float(scale)
        ctx.has_bias = bias is not None
        return dt

    @staticmethod
    def backward(ctx, ddt):
        (dt,) = ctx.saved_tensors
        b, d, l = dt.shape
        lib = _lib.load()
        ddt = ddt.contiguous()
        dpre = torch.empty_like(dt)
        dbias = torch.empty(d, device=dt.device, dtype=torch.float32) if ctx.has_bias else None
        with torch.cuda.device(dt.device):
            ws = _workspace(lib.aussm_b200_softplus_bias_bwd_workspace_bytes(b, d), dt.device)
            rc = lib.aussm_b200_softplus_bias_bwd(_ptr(ddt), _ptr(dt), ctx.scale, _ptr(dpre), _ptr(dbias), b, d, l,
                                                  _ptr(ws), ws.numel(), _stream(dt))
        _lib.check(rc, "softplus_bias backward")
        return dpre, dbias, None


def softplus_bias(pre: Tensor, bias: Tensor = None, scale: float = 1.0) -> Tensor:
    """``softplus(pre + scale * bias[None, :, None])`` for ``pre`` (b, d, l): the block's step size
    (aussm.py:878-880, where dt_proj's bias enters a second time) in one pass."""
    b, d, l = pre.shape
    return _SoftplusBias.apply(_f32c("pre", pre, (b, d, l)), None if bias is None else _f32c("bias", bias, (d,)), scale)


# ---------------------------------------------------------------------------
# linear layers with channel-major results
# ---------------------------------------------------------------------------
def _big(flop: float, *dims: int) -> bool:
    return flop >= MIN_FLOP


def _weight_grad(A: Tensor, a_mn: int, B: Tensor, b_mn: int, m: int, k: int, l: int, b: int) -> Tensor:
    """``dW[m][k] = sum_b sum_t A_b(m, t) B_b(k, t)`` for batched operands whose contraction index is time.

    ``x_mn == 0``: operand stored (rows, l) per batch entry, ``x_mn == 1``: stored (l, rows).  The output has few
    tiles and a very long contraction, so the time axis is cut into slices that run as independent batch entries
    of the split GEMM (one partial product each, through the strided entry point: the slices are views), and the
    partial products are added afterwards."""
    tiles = ((m + 127) // 128) * ((k + 255) // 256)
    slices = 1
    while tiles * slices * 2 <= 296 and l % (2 * slices) == 0 and (l // (2 * slices)) % 8 == 0 and l // (2 * slices) >= 512:
        slices *= 2
    ls = l // slices
    lib = _lib.load()
    part = torch.empty(b, slices, m, k, device=A.device, dtype=torch.float32)
    a_rows, b_rows = (m, k)
    lda, ldb = (l if a_mn == 0 else a_rows), (l if b_mn == 0 else b_rows)
    a_step = ls if a_mn == 0 else ls * a_rows           # floats between consecutive time slices
    b_step = ls if b_mn == 0 else ls * b_rows
    with torch.cuda.device(A.device):
        ws = _workspace(lib.aussm_b200_gemm_split3_workspace_bytes(m, k, ls, slices, a_mn, 1, b_mn, 1), A.device)
        for i in range(b):
            rc = lib.aussm_b200_gemm_split3_strided(
                A[i].data_ptr(), a_mn, lda, a_step, B[i].data_ptr(), b_mn, ldb, b_step, part[i].data_ptr(), k, m * k, m, k,
                ls, slices, 0, 0, _ptr(ws), ws.numel(), _stream(A))
            _lib.check(rc, "weight gradient (split GEMM)")
    return part.sum((0, 1))


class _ProjectTokens(torch.autograd.Function):
    """out[b] (m, l) = W (m, k) x[b]^T  for token-major x (b, l, k)."""

    @staticmethod
    def forward(ctx, W, x):
        m, k = W.shape
        b, l, _ = x.shape
        out = torch.empty(b, m, l, device=x.device, dtype=torch.float32)
        # A = W: (rows m, K) K-major, shared; B = x[b]: (rows l, K) K-major, batched
        _gemm(W, 0, 0, x, 0, 1, out, m, l, k, b, 0)
        ctx.save_for_backward(W, x)
        return out

    @staticmethod
    def backward(ctx, g):
        W, x = ctx.saved_tensors
        m, k = W.shape
        b, l, _ = x.shape
        g = g.contiguous()
        dW = dx = None
        if ctx.needs_input_grad[0]:
            # dW (m, k) = sum_b g[b] (m, K = l: K-major) x[b] (K = l rows, k contiguous: MN-major)
            dW = _weight_grad(g, 0, x, 1, m, k, l, b)
        if ctx.needs_input_grad[1]:
            dx = torch.empty_like(x)
            # dx[b] (l, k) = g[b]^T (l, K = m) W (K = m, k): g[b] stored (K rows, l contiguous) and W stored
            # (K rows, k contiguous): both MN-major
            _gemm(g, 1, 1, W, 1, 0, dx, l, k, m, b, 0)
        return dW, dx


def project_tokens(W: Tensor, x: Tensor) -> Tensor:
    """``einsum('mk,blk->bml')``: a linear layer applied to token-major ``x`` (b, l, k) whose result is
    channel-major (b, m, l)."""
    m, k = W.shape
    b, l, _ = x.shape
    if _big(2.0 * b * l * m * k):
        return _ProjectTokens.apply(_f32c("W", W), _f32c("x", x, (b, l, k)))
    return torch.matmul(W, x.transpose(1, 2))


def project_channels(W: Tensor, u: Tensor) -> Tensor:
    """``einsum('mk,bkl->bml')`` for channel-major ``u`` (b, k, l): result (b, m, l)."""
    m, k = W.shape
    b, _, l = u.shape
    if _big(2.0 * b * l * m * k):
        from .variants import _Projection
        return _Projection.apply(_f32c("W", W), _f32c("u", u, (b, k, l)))
    return torch.matmul(W, u)


class _ProjectBack(torch.autograd.Function):
    """out[b] (l, m) = y[b]^T (l, k) W^T  for channel-major y (b, k, l), W (m, k)."""

    @staticmethod
    def forward(ctx, W, y):
        m, k = W.shape
        b, _, l = y.shape
        out = torch.empty(b, l, m, device=y.device, dtype=torch.float32)
        # A = y[b]: (K = k rows, l contiguous) MN-major, batched; B = W: (rows m, K) K-major, shared
        _gemm(y, 1, 1, W, 0, 0, out, l, m, k, b, 0)
        ctx.save_for_backward(W, y)
        return out

    @staticmethod
    def backward(ctx, g):
        W, y = ctx.saved_tensors
        m, k = W.shape
        b, _, l = y.shape
        g = g.contiguous()
        dW = dy = None
        if ctx.needs_input_grad[0]:
            # dW (m, k) = sum_b g[b]^T (m, K = l) y[b]^T (K = l, k): g[b] stored (K = l rows, m contiguous)
            # MN-major, y[b] stored (k rows, K = l contiguous) K-major
            dW = _weight_grad(g, 1, y, 0, m, k, l, b)
        if ctx.needs_input_grad[1]:
            dy = torch.empty_like(y)
            # dy[b] (k, l) = W^T (k, K = m) g[b]^T (K = m, l): W stored (K rows, k contiguous) MN-major, shared;
            # g[b] stored (l rows, K = m contiguous) K-major
            _gemm(W, 1, 0, g, 0, 1, dy, k, l, m, b, 0)
        return dW, dy


def project_back(W: Tensor, y: Tensor, bias: Tensor = None) -> Tensor:
    """``einsum('mk,bkl->blm')`` (+ bias): a linear layer applied to channel-major ``y`` (b, k, l) whose result
    is token-major (b, l, m)."""
    m, k = W.shape
    b, _, l = y.shape
    if _big(2.0 * b * l * m * k):
        out = _ProjectBack.apply(_f32c("W", W), _f32c("y", y, (b, k, l)))
    else:
        out = torch.matmul(y.transpose(1, 2), W.t())
    return out if bias is None else out + bias
