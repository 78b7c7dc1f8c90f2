"""The callers of the scan operators: AUSSM / Mamba blocks and the two model
families the benchmark configurations use, written against this package's
operators.

These are re-statements of the reference's PyTorch modules with the SAME
parameter names and shapes, so that a reference checkpoint's ``state_dict``
loads unchanged (ai-modules/wavesAI/model/aussm.py: ``SSMTS`` :100-227,
``SSMSequenceClassifier`` :382-536, ``ResidualBlock`` :681-714, ``MambaBlock``
:717-805, ``SSMauBlock`` :808-902, ``RMSNorm`` :905-916).  Only the scan calls
differ: ``SSMauBlock`` calls ``aussm_b200.ops.ssm_adaptive_interface`` and
``MambaBlock`` calls ``aussm_b200.s6.selective_scan_fn`` (the reference imports
the latter from the third-party package mamba-ssm); and the ``nn.Linear``
layers are ``aussm_b200.linear.SplitLinear`` (same parameters; the float32
products run on the tensor cores through the library's split GEMM).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops, s6, stages
from .linear import SplitLinear, split_linear

__all__ = ["RMSNorm", "SSMauBlock", "MambaBlock", "ResidualBlock", "SSMTS", "SSMSequenceClassifier"]


class RMSNorm(nn.Module):
    def __init__(self, d_model: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(d_model))

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


def _causal_depthwise_conv(conv: nn.Conv1d, x_bld: torch.Tensor) -> torch.Tensor:
    """(b, l, d) -> (b, l, d): the block's depthwise convolution, cut back to l steps (causal)."""
    l = x_bld.shape[1]
    return conv(x_bld.transpose(1, 2))[:, :, :l].transpose(1, 2)


class SSMauBlock(nn.Module):
    """AUSSM mixer: in_proj -> depthwise conv -> adaptive unitary scan -> out_proj (aussm.py:808-902)."""

    def __init__(self, d_model: int, d_state: int, dt_rank=None, d_conv: int = 4, conv_bias: bool = True,
                 bias: bool = False, conv_1d: bool = True):
        super().__init__()
        self.d_model, self.d_state, self.use_conv = d_model, d_state, conv_1d
        dt_rank = d_state if dt_rank in (None, "auto") else dt_rank
        self.in_proj = SplitLinear(d_model, 2 * d_model, bias=bias)
        self.conv1d = nn.Conv1d(d_model, d_model, kernel_size=d_conv, groups=d_model, padding=d_conv - 1,
                                bias=conv_bias)
        self.out_proj = SplitLinear(d_model, d_model, bias=bias)
        self.x_proj = SplitLinear(d_model, dt_rank, bias=False)
        self.dt_proj = SplitLinear(dt_rank, d_model, bias=True)
        self.D = nn.Parameter(torch.ones(d_model))
        self.C = nn.Parameter(torch.randn(d_state, dtype=torch.complex64))
        self.B = nn.Parameter(torch.randn(d_state, dtype=torch.complex64))
        self.xA_proj = SplitLinear(d_model, d_model * d_state, bias=True)
        with torch.no_grad():
            self.xA_proj.bias.uniform_(-math.pi, math.pi)

    def _operator_parameters(self):
        # xA_proj's rows are ordered (state, channel): weight (n*d, d) -> x[i][j][r], bias -> x_bias[i][j]
        d, n = self.d_model, self.d_state
        x_param = self.xA_proj.weight.view(n, d, d).transpose(0, 1).contiguous() * (1.0 / math.sqrt(d))
        x_bias = self.xA_proj.bias.view(n, d).transpose(0, 1).contiguous()
        return x_param, x_bias

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.float32 and self.conv1d.kernel_size[0] <= 4:
            return self._forward_channel_major(x)
        # The reference's order of operations, token-major with transposes (aussm.py:849-902).  CUDA tensors
        # take the channel-major path below; this one is what the module-glue test pins against the reference's
        # own class on the CPU (with the oracle's scan substituted for the operator).
        b, l, d = x.shape
        xs, z = self.in_proj(x).split([d, d], dim=-1)
        if self.use_conv:
            xs = _causal_depthwise_conv(self.conv1d, xs)
        # the step size: the reference adds dt_proj's bias a second time before the softplus (aussm.py:878-880)
        dt = F.softplus(self.dt_proj(self.x_proj(xs)) + self.dt_proj.bias)
        x_param, x_bias = self._operator_parameters()
        y = ops.ssm_adaptive_interface(u=xs.transpose(1, 2).contiguous(), dt=dt.transpose(1, 2).contiguous(),
                                       x=x_param, x_bias=x_bias, B=self.B, C=self.C, D=self.D.float(),
                                       z=z.transpose(1, 2).contiguous(), unitary=True)
        return self.out_proj(y.transpose(1, 2))

    def _forward_channel_major(self, x):
        """The same block with every stage producing (b, d, l) directly: the linear layers write channel-major
        results, the convolution with its bias and the step size (softplus with the doubled bias) are one
        pass each, and no transposing copy exists on either side of the operator."""
        d = self.d_model
        w_in, b_in = self.in_proj.weight, self.in_proj.bias
        xs = stages.project_tokens(w_in[:d], x)                      # (b, d, l)
        z = stages.project_tokens(w_in[d:], x)
        if b_in is not None:
            xs = xs + b_in[:d, None]
            z = z + b_in[d:, None]
        u = stages.causal_conv_bias(xs, self.conv1d.weight, self.conv1d.bias) if self.use_conv else xs
        low = stages.project_channels(self.x_proj.weight, u)         # (b, rank, l)
        pre = stages.project_channels(self.dt_proj.weight, low)      # (b, d, l), dt_proj without its bias
        dt = stages.softplus_bias(pre, self.dt_proj.bias, 2.0)       # the bias enters twice (aussm.py:878-880)
        x_param, x_bias = self._operator_parameters()
        y = ops.ssm_adaptive_interface(u=u, dt=dt, x=x_param, x_bias=x_bias, B=self.B, C=self.C, D=self.D.float(),
                                       z=z, unitary=True)
        return stages.project_back(self.out_proj.weight, y, self.out_proj.bias)


class MambaBlock(nn.Module):
    """Mamba (S6) mixer (aussm.py:717-805)."""

    def __init__(self, d_model: int, d_state: int = 16, expand: int = 2, dt_rank=None, d_conv: int = 4,
                 conv_bias: bool = True, bias: bool = False):
        super().__init__()
        self.d_model, self.d_state = d_model, d_state
        self.d_inner = int(expand * d_model)
        self.dt_rank = math.ceil(d_model / 16) if dt_rank in (None, "auto") else dt_rank
        self.in_proj = SplitLinear(d_model, 2 * self.d_inner, bias=bias)
        self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, kernel_size=d_conv, groups=self.d_inner,
                                padding=d_conv - 1, bias=conv_bias)
        self.out_proj = SplitLinear(self.d_inner, d_model, bias=bias)
        self.x_proj = SplitLinear(self.d_inner, self.dt_rank + 2 * d_state, bias=False)
        self.dt_proj = SplitLinear(self.dt_rank, self.d_inner, bias=True)
        self.D = nn.Parameter(torch.ones(self.d_inner))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, d_state + 1, dtype=torch.float32)).repeat(self.d_inner, 1))
        self.A_log._no_weight_decay = True

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.float32 and self.conv1d.kernel_size[0] <= 4:
            return self._forward_channel_major(x)
        # the reference's token-major order of operations (aussm.py:749-805); see SSMauBlock.forward
        di, n = self.d_inner, self.d_state
        xs, z = self.in_proj(x).split([di, di], dim=-1)
        xs = _causal_depthwise_conv(self.conv1d, xs)
        dt, Bm, Cm = self.x_proj(xs).split([self.dt_rank, n, n], dim=-1)
        # dt_proj is applied with its bias, and the bias goes in once more as delta_bias (aussm.py:786-799)
        y = s6.selective_scan_fn(F.silu(xs).transpose(1, 2).contiguous(), self.dt_proj(dt).transpose(1, 2).contiguous(),
                                 (-torch.exp(self.A_log.float())).contiguous(), Bm.transpose(1, 2).contiguous(),
                                 Cm.transpose(1, 2).contiguous(), self.D.float().contiguous(),
                                 z=z.transpose(1, 2).contiguous(), delta_bias=self.dt_proj.bias.float(),
                                 delta_softplus=True)
        return self.out_proj(y.transpose(1, 2))


    def _forward_channel_major(self, x):
        """Channel-major form of the block (see SSMauBlock._forward_channel_major)."""
        di, n, r = self.d_inner, self.d_state, self.dt_rank
        w_in, b_in = self.in_proj.weight, self.in_proj.bias
        xs = stages.project_tokens(w_in[:di], x)
        z = stages.project_tokens(w_in[di:], x)
        if b_in is not None:
            xs = xs + b_in[:di, None]
            z = z + b_in[di:, None]
        xs = stages.causal_conv_bias(xs, self.conv1d.weight, self.conv1d.bias)
        low = stages.project_channels(self.x_proj.weight, xs)       # (b, rank + 2n, l): dt, B, C rows
        dt = stages.project_channels(self.dt_proj.weight, low[:, :r].contiguous()) + self.dt_proj.bias[:, None]
        # dt_proj is applied with its bias, and the bias goes in once more as delta_bias (aussm.py:786-799)
        y = s6.selective_scan_fn(F.silu(xs), dt, (-torch.exp(self.A_log.float())).contiguous(),
                                 low[:, r:r + n].contiguous(), low[:, r + n:].contiguous(),
                                 self.D.float().contiguous(), z=z, delta_bias=self.dt_proj.bias.float(),
                                 delta_softplus=True)
        return stages.project_back(self.out_proj.weight, y, self.out_proj.bias)


class ResidualBlock(nn.Module):
    """x + mixer(norm(x))."""

    def __init__(self, mixer: nn.Module, d_model: int):
        super().__init__()
        self.mixer = mixer
        self.norm = RMSNorm(d_model)

    def forward(self, x):
        return self.mixer(self.norm(x)) + x


def _build_layers(layers: str, d_model, d_state, mamba_expand, dt_rank, d_conv, conv_bias, bias, ssmau_conv_1d):
    blocks = []
    for kind in layers.replace(" ", "").split("|"):
        if kind == "a":
            mixer = SSMauBlock(d_model, d_state, dt_rank, d_conv, conv_bias, bias, ssmau_conv_1d)
        elif kind == "m":
            mixer = MambaBlock(d_model, d_state, mamba_expand, dt_rank, d_conv, conv_bias, bias)
        else:
            raise NotImplementedError(f'Layer type "{kind}" not recognized')
        blocks.append(ResidualBlock(mixer, d_model))
    return nn.ModuleList(blocks)


class SSMTS(nn.Module):
    """Time-series model: Linear embedding -> 'a|m|...' residual blocks -> RMSNorm -> Linear head, per step."""

    def __init__(self, d_model: int, input_dim: int, output_dim: int, layers: str = "m|a", d_state: int = 16,
                 mamba_expand: int = 2, dt_rank="auto", d_conv: int = 4, conv_bias: bool = True, bias: bool = False,
                 ssmau_conv_1d: bool = True):
        super().__init__()
        self.embedding = SplitLinear(input_dim, d_model)
        self.layers = _build_layers(layers, d_model, d_state, mamba_expand, dt_rank, d_conv, conv_bias, bias,
                                    ssmau_conv_1d)
        self.norm_f = RMSNorm(d_model)
        self.output = SplitLinear(d_model, output_dim, bias=False)

    def forward(self, x):
        x = self.embedding(x)
        for layer in self.layers:
            x = layer(x)
        return self.output(self.norm_f(x))


class SSMSequenceClassifier(nn.Module):
    """Token classifier: Embedding -> blocks -> pool over time ("meanpool" or "last") -> RMSNorm -> Linear."""

    def __init__(self, d_model: int, vocab_size: int, output_dim: int, layers: str = "m|a", d_state: int = 16,
                 mamba_expand: int = 2, dt_rank="auto", d_conv: int = 4, conv_bias: bool = True, bias: bool = False,
                 mode: str = "meanpool", ssmau_conv_1d: bool = True):
        super().__init__()
        self.meanpool = "meanpool" in mode
        self.embedding = nn.Embedding(vocab_size, d_model)
        self.layers = _build_layers(layers, d_model, d_state, mamba_expand, dt_rank, d_conv, conv_bias, bias,
                                    ssmau_conv_1d)
        self.norm_f = RMSNorm(d_model)
        self.output = SplitLinear(d_model, output_dim, bias=False)

    def forward(self, input_ids, lengths=None):
        x = self.embedding(input_ids)
        for layer in self.layers:
            x = layer(x)
        if lengths is not None:
            idx = torch.arange(x.shape[1], device=x.device)[None, :]
            if self.meanpool:
                mask = (idx < lengths[:, None]).to(x.dtype)[..., None]
                x = (x * mask).sum(1) / lengths[:, None].to(x.dtype)
            else:
                x = x[torch.arange(x.shape[0], device=x.device), lengths - 1]
        else:
            x = x.mean(1) if self.meanpool else x[:, -1]
        return self.output(self.norm_f(x))
