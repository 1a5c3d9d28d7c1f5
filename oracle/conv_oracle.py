"""CPU gather-matmul-scatter restatement of PCEngine's sparse convolution
(TEST INFRASTRUCTURE ONLY: imported by tests, the smoke check and the
benchmark's CPU-baseline / reference legs, never by the product package).

PARITY PINNED: tests/test_ref_golden.py compares ``conv_forward`` with the fp32
output of the reference's own ``conv_fwd_d2_cuda`` (fixtures tests/golden/ref_*.npz,
written on a B200 by tests/golden/make_ref_golden.py) at rel-L2 <= 1e-5, and with
dense ``torch.nn.functional.conv3d`` on small grids (tests/test_oracle_dense.py).

Semantics restated: script/spconv.py:291-464 (dispatch, centre offset, bias,
transposed = maps swapped), backend/spconv.cu:224-398 and the pair loop of
backend/spconv.cuh:1653-1728 (out[omap[y]] += in[imap[y]] @ W[kp]).  Arithmetic
is fp32 on the (possibly fp16-rounded) inputs, which is the accumulate type the
build requires; the reference's fp16 accumulation is not restated.
"""
from __future__ import annotations

import numpy as np
import torch

from . import kmap_oracle as ko


def conv_forward(feats: torch.Tensor, kernel: torch.Tensor, d2: dict, transposed: bool = False,
                 bias: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 sparse conv from the pair lists of ``ko.build_d2``.

    feats [N_in, C_in] (rows of the *coarse* side when transposed), kernel
    [kv, C_in, C_out].  The centre offset of a submanifold map is applied as the
    dense product the reference issues first (backend/spconv.cu:273-298).
    """
    x = feats.float()
    w = kernel.float()
    if w.dim() == 2:
        w = w[None]
    imap = torch.from_numpy(d2["imap"].astype(np.int64))
    omap = torch.from_numpy(d2["omap"].astype(np.int64))
    n_out = d2["n_out"]
    if transposed:
        imap, omap = omap, imap
        n_out = d2["n_in"]
    out = torch.zeros((n_out, w.shape[2]), dtype=torch.float32)
    if d2["subm"]:
        out += x @ w[d2["mid"]]
    kpos = d2["kpos"]
    for kp in range(d2["kv"]):
        a, b = int(kpos[kp]), int(kpos[kp + 1])
        if b > a:
            out.index_add_(0, omap[a:b], x[imap[a:b]] @ w[kp])
    if bias is not None:
        out += bias.float()
    return out


def pointwise_conv(feats, kernel, bias=None):
    """1x1x1 stride-1 shortcut, script/spconv.py:297-304."""
    out = feats.float() @ kernel.float()
    if bias is not None:
        out += bias.float()
    return out


def batchnorm_eval(x, weight, bias, mean, var, eps=1e-5):
    """Inference-mode nn.BatchNorm1d on [N, C] rows (script/batchnorm.py:7-11)."""
    scale = weight.float() / torch.sqrt(var.float() + eps)
    return (x.float() - mean.float()) * scale + bias.float()


def activation(x, kind: str = "relu", slope: float = 0.01):
    """nn.ReLU / nn.LeakyReLU on the feature rows (script/activation.py:6-15)."""
    if kind == "relu":
        return torch.relu(x)
    if kind == "leaky":
        return torch.nn.functional.leaky_relu(x, slope)
    return x


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a-b||_F / ||b||_F in float64."""
    a = a.double().cpu()
    b = b.double().cpu()
    den = float(torch.linalg.norm(b))
    num = float(torch.linalg.norm(a - b))
    return num / den if den > 0 else num
