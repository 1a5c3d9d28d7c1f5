"""A MinkUNet-shaped segmentation network composed from the operator surface
(conv3d / BatchNorm / ReLU / cat and residual adds).  The reference ships no model;
this one follows the description it is benchmarked on: a 3x3x3 submanifold stem,
four encoder stages (2x2x2 stride-2 down conv, then two residual 3x3x3 blocks), four
decoder stages (transposed 2x2x2 up conv, skip concatenation, two residual blocks)
and a 1x1x1 classifier.  Widths: stem 32; encoder 32, 64, 128, 256; decoder 256, 128,
96, 96 (the width list 32-64-128-256-256-128-96-96 scaled by ``cr``).

In eval mode on a CUDA tensor every BatchNorm + ReLU (+ residual add) is folded into
the producing convolution's epilogue; in training mode or on CPU tensors the plain
modules run.
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from .activation import ReLU
from .batchnorm import BatchNorm, bn_scale_shift
from .functional import FusedEpilogue, supports_second_operand
from .planner import MapPlan
from .spconv import conv3d, conv_func
from .sptensor import spTensor
from .utils import cat


class _Fusable(nn.Module):
    """Caches folded BatchNorm constants while the module stays in eval mode."""

    def __init__(self):
        super().__init__()
        self._folded = {}

    def train(self, mode: bool = True):
        self._folded = {}
        return super().train(mode)

    def _apply(self, fn, *args, **kwargs):
        self._folded = {}
        return super()._apply(fn, *args, **kwargs)

    def _fold(self, name: str, bn: nn.BatchNorm1d):
        if name not in self._folded:
            self._folded[name] = bn_scale_shift(bn)
        return self._folded[name]

    def _fold_weight(self, name: str, weight: torch.Tensor, scale: torch.Tensor, dtype):
        """``weight`` [..., C_out] times the per-channel BatchNorm scale, in ``dtype`` (cached like
        the folded constants; the tensor-core layout is cached on the result)."""
        key = (name, dtype)
        if key not in self._folded:
            self._folded[key] = (weight.detach().float() * scale).to(dtype).contiguous()
        return self._folded[key]

    def _fused(self, x: spTensor) -> bool:
        return (not self.training) and x.feats.is_cuda


class ConvBNReLU(_Fusable):
    def __init__(self, cin, cout, ks=3, stride=1, transposed=False):
        super().__init__()
        self.conv = conv3d(cin, cout, ks, stride, transposed=transposed)
        self.bn = BatchNorm(cout)
        self.relu = ReLU(True)

    def forward(self, x: spTensor, out: Optional[torch.Tensor] = None) -> spTensor:
        """``out`` (fused path only): the tensor the output features are written into."""
        if self._fused(x):
            s, t = self._fold("bn", self.bn)
            return self.conv(x, epilogue=FusedEpilogue(scale=s, shift=t, act="relu"), out=out)
        return self.relu(self.bn(self.conv(x)))


class ResidualBlock(_Fusable):
    # fold the shortcut into conv2's launch when the tensor-core kernel can take it
    one_kernel_tail = True

    def __init__(self, cin, cout, ks=3):
        super().__init__()
        self.conv1 = conv3d(cin, cout, ks, 1)
        self.bn1 = BatchNorm(cout)
        self.conv2 = conv3d(cout, cout, ks, 1)
        self.bn2 = BatchNorm(cout)
        self.relu = ReLU(True)
        if cin != cout:
            self.short_conv = conv3d(cin, cout, 1, 1)
            self.short_bn = BatchNorm(cout)
        else:
            self.short_conv = None
            self.short_bn = None

    def _one_kernel_tail(self, x: spTensor, y: spTensor, out: Optional[torch.Tensor] = None) -> spTensor:
        """relu(bn2(conv2(y)) + shortcut(x)) as ONE convolution launch: both BatchNorm scales are
        folded into the weights, and the shortcut (its 1x1x1 convolution, or the identity) enters the
        accumulator as the second operand of conv2."""
        c2, dtype = self.conv2, x.feats.dtype
        s2, t2 = self._fold("bn2", self.bn2)
        w_main = self._fold_weight("conv2", c2.kernel, s2, dtype)
        if self.short_conv is not None:
            ss, ts = self._fold("short_bn", self.short_bn)
            w_extra = self._fold_weight("short", self.short_conv.kernel, ss, dtype)
            if "shift_sum" not in self._folded:
                self._folded["shift_sum"] = (t2 + ts).contiguous()
            shift = self._folded["shift_sum"]
        else:
            key = ("eye", dtype)
            if key not in self._folded:
                self._folded[key] = torch.eye(c2.out_channels, dtype=dtype, device=x.feats.device)
            w_extra, shift = self._folded[key], t2
        ep = FusedEpilogue(shift=shift, act="relu", extra_feats=x.feats.contiguous(), extra_weight=w_extra)
        return conv_func(input=y, in_channel=c2.in_channels, out_channel=c2.out_channels, kernel=w_main,
                         kernel_size_code=c2.kernel_size_code, stride_code=c2.stride_code, padding_code=c2.padding_code,
                         bias=None, transposed=False, tensorcore=c2.tensorcore, epilogue=ep, out=out)

    def forward(self, x: spTensor, out: Optional[torch.Tensor] = None) -> spTensor:
        """``out`` (fused path only): the tensor the block's output features are written into."""
        if self._fused(x):
            s1, t1 = self._fold("bn1", self.bn1)
            y = self.conv1(x, epilogue=FusedEpilogue(scale=s1, shift=t1, act="relu"))
            if (self.one_kernel_tail and self.conv2.bias is None and self.conv2.kernel_volume <= 128
                    and (self.short_conv is None or self.short_conv.bias is None)
                    and supports_second_operand(x.feats.dtype, self.conv2.in_channels, self.conv2.out_channels,
                                                x.feats.size(1))):
                return self._one_kernel_tail(x, y, out)
            if self.short_conv is not None:
                ss, ts = self._fold("short_bn", self.short_bn)
                sc = self.short_conv(x, epilogue=FusedEpilogue(scale=ss, shift=ts)).feats
            else:
                sc = x.feats.contiguous()
            s2, t2 = self._fold("bn2", self.bn2)
            return self.conv2(y, epilogue=FusedEpilogue(scale=s2, shift=t2, residual=sc, act="relu"), out=out)
        y = self.bn2(self.conv2(self.relu(self.bn1(self.conv1(x)))))
        sc = x if self.short_conv is None else self.short_bn(self.short_conv(x))
        return self.relu(y + sc)


class MinkUNet(nn.Module):
    def __init__(self, in_channels: int = 4, num_classes: int = 19, cr: float = 1.0):
        super().__init__()
        cs = [int(cr * c) for c in (32, 32, 64, 128, 256, 256, 128, 96, 96)]
        self.widths = cs
        self.in_channels = in_channels
        self.stem = nn.Sequential(ConvBNReLU(in_channels, cs[0], 3), ConvBNReLU(cs[0], cs[0], 3))
        self.down = nn.ModuleList()
        self.enc = nn.ModuleList()
        for i in range(4):
            self.down.append(ConvBNReLU(cs[i], cs[i], 2, 2))
            self.enc.append(nn.Sequential(ResidualBlock(cs[i], cs[i + 1]), ResidualBlock(cs[i + 1], cs[i + 1])))
        self.up = nn.ModuleList()
        self.dec = nn.ModuleList()
        skips = [cs[3], cs[2], cs[1], cs[0]]
        for i in range(4):
            self.up.append(ConvBNReLU(cs[4 + i], cs[5 + i], 2, 2, transposed=True))
            self.dec.append(nn.Sequential(ResidualBlock(cs[5 + i] + skips[i], cs[5 + i]),
                                          ResidualBlock(cs[5 + i], cs[5 + i])))
        self.classifier = conv3d(cs[8], num_classes, 1, 1, bias=True)

    def layer_plan(self) -> list:
        """The convolutions in forward order as (kernel_size, stride, transposed, C_in, C_out), one
        entry per distinct use of a kernel map (what :class:`MapPlan` takes)."""
        cs = self.widths
        skips = [cs[3], cs[2], cs[1], cs[0]]
        plan = [(3, 1, False, self.in_channels, cs[0]), (3, 1, False, cs[0], cs[0])]
        for i in range(4):
            plan += [(2, 2, False, cs[i], cs[i]), (3, 1, False, cs[i], cs[i + 1]), (3, 1, False, cs[i + 1], cs[i + 1])]
        for i in range(4):
            plan += [(2, 2, True, cs[4 + i], cs[5 + i]), (3, 1, False, cs[5 + i] + skips[i], cs[5 + i]),
                     (3, 1, False, cs[5 + i], cs[5 + i])]
        return plan

    # Hand the kernel maps of a pass to the library's planning thread (eval mode, CUDA) instead of
    # building each one inside the layer that first needs it.
    plan_ahead = True

    def plan(self, x: spTensor) -> bool:
        """Start building the kernel maps of ``x``'s pass now (eval mode, CUDA) and attach the pass to
        ``x``; ``forward(x)`` then finds it started.  A serving loop calls this as soon as a batch's
        coordinates are on their way to the device (``x.coords_ready``), before it runs the batch in front
        of it, so that no layer waits for a map.  Returns False when nothing was started."""
        if not self.plan_ahead or self.training or not x.feats.is_cuda or x.planner is not None:
            return False
        plans = self.__dict__.setdefault("_map_plans", {})
        plan = plans.get(x.feats.dtype)
        if plan is None:
            plan = plans[x.feats.dtype] = MapPlan(self.layer_plan(), x.stride, x.feats.dtype)
        return plan.begin(x)

    def forward(self, x: spTensor) -> spTensor:
        self.plan(x)
        if self.shared_skip_buffers and not self.training and x.feats.is_cuda and x.feats.dtype == torch.float16:
            return self._forward_shared(x)
        feats: List[spTensor] = [self.stem(x)]
        for i in range(4):
            feats.append(self.enc[i](self.down[i](feats[-1])))
        y = feats[4]
        for i in range(4):
            y = self.up[i](y)
            y = self.dec[i](cat([y, feats[3 - i]]))
        return self.classifier(y)

    # Inference in fp16: every decoder stage's input [up-sampled | skip] is ONE matrix that the
    # encoder's skip layer and the up-sampling layer write their column ranges of, instead of a
    # concatenation pass over both.
    shared_skip_buffers = True

    def _forward_shared(self, x: spTensor) -> spTensor:
        cs = self.widths
        joined: List[torch.Tensor] = []   # per encoder level: [rows, C_up + C_skip]

        def skip_view(rows: int, level: int) -> torch.Tensor:
            c_up, c_skip = cs[8 - level], cs[level]
            buf = torch.empty((rows, c_up + c_skip), dtype=x.feats.dtype, device=x.feats.device)
            joined.append(buf)
            return buf[:, c_up:]

        h = self.stem[0](x)
        y = self.stem[1](h, out=skip_view(h.feats.size(0), 0))
        for i in range(4):
            d = self.down[i](y)
            h = self.enc[i][0](d)
            y = self.enc[i][1](h, out=skip_view(h.feats.size(0), i + 1) if i < 3 else None)
        for i in range(4):
            level = 3 - i
            c_up = cs[5 + i]
            u = self.up[i](y, out=joined[level][:, :c_up])
            y = self.dec[i](u._like(joined[level]))
        return self.classifier(y)

    @staticmethod
    def tags() -> list:
        """Dataflow tags for the nine kernel maps a forward pass builds (five submanifold
        resolutions, four down-sampling layers; the transposed layers reuse those)."""
        return ["auto"]


def randomize_batchnorm(model: nn.Module, seed: int = 0) -> None:
    """Give every BatchNorm non-trivial running statistics and affine terms (seeded), so a
    randomly initialised network exercises the fused epilogues."""
    g = torch.Generator().manual_seed(seed)
    for m in model.modules():
        if isinstance(m, nn.BatchNorm1d):
            n = m.num_features
            m.running_mean.copy_((torch.rand(n, generator=g) - 0.5) * 0.2)
            m.running_var.copy_(0.8 + 0.4 * torch.rand(n, generator=g))
            m.weight.data.copy_(0.8 + 0.4 * torch.rand(n, generator=g))
            m.bias.data.copy_((torch.rand(n, generator=g) - 0.5) * 0.2)
    for m in model.modules():
        if isinstance(m, _Fusable):
            m._folded = {}  # constants folded from the old statistics
