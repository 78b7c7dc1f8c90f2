"""The block-stage kernels and channel-major projections against their eager PyTorch definitions
(the reference block's own sequence of operations, ai-modules/wavesAI/model/aussm.py:849-902), and the
channel-major block paths against the token-major ones."""
import pytest
import torch
import torch.nn.functional as F

import aussm_b200
from aussm_b200 import models, stages
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,k", [((2, 6, 40), 4), ((1, 3, 7), 4), ((3, 16, 128), 3), ((2, 5, 33), 2), ((1, 4, 1), 4),
                                     ((2, 128, 720), 4)])
@pytest.mark.parametrize("with_bias", [True, False])
def test_causal_conv_bias_matches_conv1d(shape, k, with_bias):
    b, d, l = shape
    g = torch.Generator().manual_seed(sum(shape) + k)
    xs = torch.randn(b, d, l, generator=g)
    w = torch.randn(d, 1, k, generator=g)
    bias = torch.randn(d, generator=g) if with_bias else None
    gy = torch.randn(b, d, l, generator=g)

    def ref(dtype):
        a = [t.to(dtype).requires_grad_(True) if t is not None else None for t in (xs, w, bias)]
        y = F.conv1d(a[0], a[1], a[2], padding=k - 1, groups=d)[..., :l]
        (y * gy.to(dtype)).sum().backward()
        return y.detach(), [t.grad if t is not None else None for t in a]

    y64, g64 = ref(torch.float64)
    a = [t.cuda().requires_grad_(True) if t is not None else None for t in (xs, w, bias)]
    y = stages.causal_conv_bias(*a)
    (y * gy.cuda()).sum().backward()
    assert_parity("u", y, y64, scaled_tol=1e-6)
    for name, t, r in zip(("xs", "weight", "bias"), a, g64):
        if t is not None:
            assert_parity("grad_" + name, t.grad, r, atol=1e-5 * float(r.abs().max()) + 1e-9, rtol=1e-3, scaled_tol=1e-5)


@pytest.mark.parametrize("shape", [(2, 6, 40), (1, 3, 7), (2, 128, 720)])
def test_softplus_bias_matches_eager(shape):
    b, d, l = shape
    g = torch.Generator().manual_seed(sum(shape))
    pre = torch.randn(b, d, l, generator=g) * 8          # both sides of the softplus threshold
    pre[0, 0, 0] = 25.0
    pre[0, 0, min(1, l - 1)] = -30.0
    bias = torch.randn(d, generator=g)
    gy = torch.randn(b, d, l, generator=g)
    p64, b64 = pre.double().requires_grad_(True), bias.double().requires_grad_(True)
    ref = F.softplus(p64 + 2.0 * b64[None, :, None])
    (ref * gy.double()).sum().backward()
    p, bb = pre.cuda().requires_grad_(True), bias.cuda().requires_grad_(True)
    out = stages.softplus_bias(p, bb, 2.0)
    (out * gy.cuda()).sum().backward()
    assert_parity("dt", out, ref.detach(), scaled_tol=1e-6)
    assert_parity("grad_pre", p.grad, p64.grad, atol=1e-6 * float(p64.grad.abs().max()), rtol=1e-4, scaled_tol=1e-6)
    assert_parity("grad_bias", bb.grad, b64.grad, atol=1e-5 * float(b64.grad.abs().max()), rtol=1e-3, scaled_tol=1e-5)


@pytest.mark.parametrize("big", [False, True])
def test_channel_major_projections_match_einsum(big):
    old = stages.MIN_FLOP
    stages.MIN_FLOP = 0.0 if big else 1e30            # force the split GEMM / the torch.matmul path
    try:
        g = torch.Generator().manual_seed(4)
        b, l, k, m = 2, 72, 24, 40
        W, x, u = torch.randn(m, k, generator=g), torch.randn(b, l, k, generator=g), torch.randn(b, k, l, generator=g)
        cases = [("tokens", stages.project_tokens, x, "mk,blk->bml"), ("channels", stages.project_channels, u, "mk,bkl->bml"),
                 ("back", stages.project_back, u, "mk,bkl->blm")]
        for name, fn, inp, eq in cases:
            W64, i64 = W.double().requires_grad_(True), inp.double().requires_grad_(True)
            ref = torch.einsum(eq, W64, i64)
            gy = torch.randn(ref.shape, generator=g)
            (ref * gy.double()).sum().backward()
            Wd, idv = W.cuda().requires_grad_(True), inp.cuda().requires_grad_(True)
            out = fn(Wd, idv)
            (out * gy.cuda()).sum().backward()
            assert_parity(name, out, ref.detach(), scaled_tol=3e-6)
            assert_parity(name + " grad_W", Wd.grad, W64.grad, scaled_tol=3e-6)
            assert_parity(name + " grad_in", idv.grad, i64.grad, scaled_tol=3e-6)
    finally:
        stages.MIN_FLOP = old
    assert aussm_b200.device_status() == 0


@pytest.mark.parametrize("kind", ["a", "m"])
def test_channel_major_block_equals_token_major_block(kind):
    """The block as the reference orders it (token-major, transposes, nn.Conv1d, separate softplus) and the
    channel-major form compute the same function and the same gradients."""
    torch.manual_seed(7)
    blk = (models.SSMauBlock(32, 8) if kind == "a" else models.MambaBlock(32, 8)).cuda()
    x = torch.randn(2, 80, 32, device="cuda")
    gy = torch.randn(2, 80, 32, device="cuda")

    def run(fast):
        for p in blk.parameters():
            p.grad = None
        xi = x.clone().requires_grad_(True)
        out = blk._forward_channel_major(xi) if fast else _token_major(blk, xi)
        (out * gy).sum().backward()
        return out.detach(), xi.grad, {k: p.grad.clone() for k, p in blk.named_parameters()}

    o1, gx1, gp1 = run(True)
    o0, gx0, gp0 = run(False)
    scale = lambda t: float(t.abs().max()) + 1e-30
    assert float((o1 - o0).abs().max()) <= 2e-5 * scale(o0)
    assert float((gx1 - gx0).abs().max()) <= 1e-4 * scale(gx0)
    for k in gp0:
        a, bb = gp1[k], gp0[k]
        if a.is_complex():
            a, bb = torch.view_as_real(a), torch.view_as_real(bb)
        assert float((a - bb).abs().max()) <= 2e-4 * scale(bb), k


def _token_major(blk, x):
    """The reference's order of operations on CUDA tensors (what forward() runs for non-CUDA input)."""
    import math
    if isinstance(blk, models.SSMauBlock):
        b, l, d = x.shape
        xs, z = blk.in_proj(x).split([d, d], dim=-1)
        xs = models._causal_depthwise_conv(blk.conv1d, xs)
        dt = F.softplus(blk.dt_proj(blk.x_proj(xs)) + blk.dt_proj.bias)
        x_param, x_bias = blk._operator_parameters()
        y = aussm_b200.ssm_adaptive_interface(u=xs.transpose(1, 2).contiguous(), dt=dt.transpose(1, 2).contiguous(),
                                              x=x_param, x_bias=x_bias, B=blk.B, C=blk.C, D=blk.D.float(),
                                              z=z.transpose(1, 2).contiguous(), unitary=True)
        return blk.out_proj(y.transpose(1, 2))
    di, n = blk.d_inner, blk.d_state
    xs, z = blk.in_proj(x).split([di, di], dim=-1)
    xs = models._causal_depthwise_conv(blk.conv1d, xs)
    dt, Bm, Cm = blk.x_proj(xs).split([blk.dt_rank, n, n], dim=-1)
    y = aussm_b200.selective_scan_fn(F.silu(xs).transpose(1, 2).contiguous(), blk.dt_proj(dt).transpose(1, 2).contiguous(),
                                     (-torch.exp(blk.A_log.float())).contiguous(), Bm.transpose(1, 2).contiguous(),
                                     Cm.transpose(1, 2).contiguous(), blk.D.float().contiguous(),
                                     z=z.transpose(1, 2).contiguous(), delta_bias=blk.dt_proj.bias.float(),
                                     delta_softplus=True)
    return blk.out_proj(y.transpose(1, 2))
