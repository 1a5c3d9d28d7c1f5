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
from . import functional as PF
from .functional import FusedEpilogue, supports_second_operand
from .netprogram import INPUT, OUTPUT, NetProgram
from .planner import MapPlan
from .spconv import conv3d, conv_func
from .sptensor import spTensor
from .utils import cat, output_stride_compute


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

    def _tail_operands(self, dtype, device):
        """(conv2's weights with bn2's scale folded in, the shortcut as a [C_in, C_out] matrix -- its
        1x1x1 convolution with its BatchNorm scale folded in, or the identity --, the summed shifts):
        the operands of the block's one-launch tail, cached while the module stays in eval mode."""
        c2 = self.conv2
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
                self._folded[key] = torch.eye(c2.out_channels, dtype=dtype, device=device)
            w_extra, shift = self._folded[key], t2
        return w_main, w_extra, shift

    def _tail_in_one_launch(self, dtype, c_x: int) -> bool:
        return (self.one_kernel_tail and self.conv2.bias is None and self.conv2.kernel_volume <= 128
                and (self.short_conv is None or self.short_conv.bias is None)
                and supports_second_operand(dtype, self.conv2.in_channels, self.conv2.out_channels, c_x))

    def _one_kernel_tail(self, x: spTensor, y: spTensor, out: Optional[torch.Tensor] = None) -> spTensor:
        """relu(bn2(conv2(y)) + shortcut(x)) as ONE convolution launch: both BatchNorm scales are
        folded into the weights, and the shortcut (its 1x1x1 convolution, or the identity) enters the
        accumulator as the second operand of conv2."""
        c2 = self.conv2
        w_main, w_extra, shift = self._tail_operands(x.feats.dtype, x.feats.device)
        ep = FusedEpilogue(shift=shift, act="relu", extra_feats=x.feats.contiguous(), extra_weight=w_extra)
        return conv_func(input=y, in_channel=c2.in_channels, out_channel=c2.out_channels, kernel=w_main,
                         kernel_size_code=c2.kernel_size_code, stride_code=c2.stride_code, padding_code=c2.padding_code,
                         bias=None, transposed=False, tensorcore=c2.tensorcore, epilogue=ep, out=out)

    def forward(self, x: spTensor, out: Optional[torch.Tensor] = None) -> spTensor:
        """``out`` (fused path only): the tensor the block's output features are written into."""
        if self._fused(x):
            s1, t1 = self._fold("bn1", self.bn1)
            y = self.conv1(x, epilogue=FusedEpilogue(scale=s1, shift=t1, act="relu"))
            if self._tail_in_one_launch(x.feats.dtype, x.feats.size(1)):
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
        if x.slabs is not None:  # one rank's slab of a scene: its submanifold maps span halo rows (spconv.conv_func)
            return False
        plans = self.__dict__.setdefault("_map_plans", {})
        plan = plans.get(x.feats.dtype)
        if plan is None:
            plan = plans[x.feats.dtype] = MapPlan(self.layer_plan(), x.stride, x.feats.dtype)
        return plan.begin(x)

    def forward(self, x: spTensor) -> spTensor:
        self.plan(x)
        if (self.shared_skip_buffers and not self.training and x.feats.is_cuda and x.feats.dtype == torch.float16
                and x.slabs is None):
            if self.one_call and x.planner is not None and not x.kmaps and PF.PROFILE is None:
                prog = self._program(x)
                if prog is not None:
                    return self._forward_program(x, prog)
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

    # Inference in fp16 with planned maps: the whole pass is ONE call into the library (NetProgram)
    # instead of one Python round trip per layer.  Same launches in the same order, bit-identical.
    one_call = True

    def train(self, mode: bool = True):
        self.__dict__.pop("_programs", None)
        return super().train(mode)

    def _apply(self, fn, *args, **kwargs):
        self.__dict__.pop("_programs", None)
        return super()._apply(fn, *args, **kwargs)

    def _program(self, x: spTensor) -> Optional[NetProgram]:
        """The pass as a NetProgram for ``x``'s dtype / device / stride (built once; None when a layer
        does not fit the one-call path, e.g. widths the tensor-core kernel does not cover)."""
        progs = self.__dict__.setdefault("_programs", {})
        key = (x.feats.dtype, x.feats.device, x.stride)
        if key not in progs:
            try:
                progs[key] = self._build_program(x.planner.plan, x.feats.dtype, x.feats.device)
            except (NotImplementedError, KeyError, ValueError):
                progs[key] = None
        return progs[key]

    def _build_program(self, plan: MapPlan, dtype, device) -> NetProgram:
        cs = self.widths
        P = NetProgram(dtype)
        strides = [plan.in_stride]
        for i in range(4):
            strides.append(output_stride_compute(self.down[i].conv.stride_code, strides[-1], 0))

        def map_of(conv, level):  # level: the FINE side of the layer's map
            return plan.index[(conv.kernel_size_code, strides[level], conv.stride_code)]

        def kernel_of(conv):
            c_in, c_out = conv.kernel.shape[-2:]
            k = conv.kernel if conv.kernel.dim() == 3 else conv.kernel.unsqueeze(0)
            if c_in % 16 or c_out % 16:
                k = PF._padded_kernel(conv.kernel, PF._ceil16(c_in), PF._ceil16(c_out))
                k = k if k.dim() == 3 else k.unsqueeze(0)
            return k

        def conv_bn_relu(m, level, src, dst, transposed=False):
            if m.conv.bias is not None:
                raise NotImplementedError
            s, t = m._fold("bn", m.bn)
            P.conv(map_of(m.conv, level), transposed, kernel_of(m.conv), src, dst, scale=s, shift=t, act="relu")

        scratch = {}

        def tmp(level, width):  # a block's intermediate: dead after the block's second layer, so shared per shape
            if (level, width) not in scratch:
                scratch[(level, width)] = P.buffer(level, width)
            return scratch[(level, width)]

        def block(m, level, src_buf, dst):
            c_x = P.buffers[src_buf][1]
            if m.conv1.bias is not None or not m._tail_in_one_launch(dtype, c_x) or c_x != m.conv1.in_channels:
                raise NotImplementedError
            s1, t1 = m._fold("bn1", m.bn1)
            mid = tmp(level, m.conv1.out_channels)
            P.conv(map_of(m.conv1, level), False, kernel_of(m.conv1), (src_buf, 0), (mid, 0), scale=s1, shift=t1, act="relu")
            w_main, w_extra, shift = m._tail_operands(dtype, device)
            P.conv(map_of(m.conv2, level), False, w_main, (mid, 0), dst, shift=shift, act="relu", extra=src_buf,
                   extra_weight=w_extra)

        joined = {}
        for level in range(4):
            joined[level] = P.buffer(level, cs[8 - level] + cs[level])  # [up-sampled | skip]
        h = P.buffer(0, cs[0])
        conv_bn_relu(self.stem[0], 0, (INPUT, 0), (h, 0))
        conv_bn_relu(self.stem[1], 0, (h, 0), (joined[0], cs[8]))
        y = (joined[0], cs[8])
        for i in range(4):
            d = P.buffer(i + 1, cs[i])
            conv_bn_relu(self.down[i], i, y, (d, 0))
            h = P.buffer(i + 1, cs[i + 1])
            block(self.enc[i][0], i + 1, d, (h, 0))
            if i < 3:
                y = (joined[i + 1], cs[8 - (i + 1)])
            else:
                y = (P.buffer(4, cs[4]), 0)
            block(self.enc[i][1], i + 1, h, y)
        for i in range(4):
            level = 3 - i
            conv_bn_relu(self.up[i], level, y, (joined[level], 0), transposed=True)
            h = P.buffer(level, cs[5 + i])
            block(self.dec[i][0], level, joined[level], (h, 0))
            y = (P.buffer(level, cs[5 + i]), 0)
            block(self.dec[i][1], level, h, y)
        head = self.classifier
        w = kernel_of(head)[0]
        shift = None
        if head.bias is not None:
            b = head.bias.detach().float()
            shift = torch.cat([b, b.new_zeros((w.size(1) - b.numel(),))]).contiguous()
        P.linear(w, y, (OUTPUT, 0), shift=shift)
        P.in_width, P.out_width = PF._ceil16(self.in_channels), w.size(1)
        P.out_channels = head.out_channels
        return P

    def _forward_program(self, x: spTensor, prog: NetProgram) -> spTensor:
        feats = x.feats
        n, c = feats.shape
        if c != prog.in_width:  # the stem's input channels, zero-padded to the kernel's granularity
            feats = torch.cat([feats, feats.new_zeros((n, prog.in_width - c))], dim=1)
        elif not feats.is_contiguous():
            feats = feats.contiguous()
        out = torch.empty((n, prog.out_width), dtype=feats.dtype, device=feats.device)
        arena = torch.empty((prog.arena_bytes(n),), dtype=torch.uint8, device=feats.device)
        handle = x.planner._handle
        prog.run(handle.handle, feats, out, arena)
        handle.stream = PF._lib.stream_ptr(feats.device)
        logits = out if prog.out_width == prog.out_channels else out[:, :prog.out_channels].contiguous()
        y = x._like(logits)
        y.kmaps = x.kmaps = _LazyMaps(x.planner)
        y.cbook = x.cbook = _LazyMaps(x.planner, book=True)
        return y

    @staticmethod
    def tags() -> list:
        """Dataflow tags for the nine kernel maps a forward pass builds (five submanifold
        resolutions, four down-sampling layers; the transposed layers reuse those)."""
        return ["auto"]


class _LazyMaps(dict):
    """``kmaps`` / ``cbook`` of a tensor whose pass ran as one library call: the planner holds the maps,
    and the dictionary the layer-by-layer path would have filled is materialised on first access."""

    def __init__(self, planner, book: bool = False):
        super().__init__()
        # the planner pass only (not the tensor): no reference cycle, so the pass is released by reference
        # counting as soon as the last tensor of the pass goes away
        self._planner, self._book, self._filled = planner, book, False

    def _fill(self):
        if self._filled:
            return
        self._filled = True
        planner, self._planner = self._planner, None

        class _Holder:
            kmaps, cbook = {}, {}

        holder = _Holder()
        holder.kmaps, holder.cbook = {}, {}
        for key, idx in planner.plan.index.items():
            planner.fetch(holder, key, planner.plan.specs[idx]["out_stride"])
        dict.update(self, holder.cbook if self._book else holder.kmaps)

    def __getitem__(self, k):
        self._fill()
        return dict.__getitem__(self, k)

    def get(self, k, default=None):
        self._fill()
        return dict.get(self, k, default)

    def __contains__(self, k):
        self._fill()
        return dict.__contains__(self, k)

    def __iter__(self):
        self._fill()
        return dict.__iter__(self)

    def __len__(self):
        self._fill()
        return dict.__len__(self)

    def __bool__(self):
        return len(self) > 0

    def keys(self):
        self._fill()
        return dict.keys(self)

    def values(self):
        self._fill()
        return dict.values(self)

    def items(self):
        self._fill()
        return dict.items(self)


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
        m.__dict__.pop("_programs", None)
