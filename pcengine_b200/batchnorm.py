"""``BatchNorm`` over the feature rows of an spTensor (script/batchnorm.py:7-11).
In eval mode the normalisation is one fused scale/shift pass of the engine, and
:func:`bn_scale_shift` exposes the folded constants so a convolution can apply
them in its epilogue instead."""
from __future__ import annotations

import torch
from torch import nn

from . import functional as PF
from .functional import FusedEpilogue
from .sptensor import spTensor
from .utils import fapply


def bn_scale_shift(bn: nn.BatchNorm1d):
    """fp32 (scale, shift) with y = x*scale + shift equal to eval-mode BatchNorm1d."""
    var = bn.running_var.detach().float()
    mean = bn.running_mean.detach().float()
    gamma = bn.weight.detach().float() if bn.affine else torch.ones_like(var)
    beta = bn.bias.detach().float() if bn.affine else torch.zeros_like(var)
    scale = gamma / torch.sqrt(var + bn.eps)
    return scale.contiguous(), (beta - mean * scale).contiguous()


class BatchNorm(nn.BatchNorm1d):

    def forward(self, input: spTensor) -> spTensor:
        if self.training or not self.track_running_stats or not input.feats.is_cuda:
            return fapply(input, super().forward)
        scale, shift = bn_scale_shift(self)
        return fapply(input, PF.scale_shift_act, FusedEpilogue(scale=scale, shift=shift))
