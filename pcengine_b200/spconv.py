"""``conv3d`` and ``conv_func``: the sparse-convolution operator
(counterpart of script/spconv.py; forward / inference only).

Dispatch follows script/spconv.py:291-464: a 1x1x1 stride-1 layer is a dense
product; a transposed layer reuses the kernel map its matching strided layer
registered, with the two sides swapped; anything else builds (or fetches) the
map keyed by (kernel-size code, tensor-stride code, layer-stride code).
Differences, all on the host: the map is a :class:`KernelMap` object instead of
a list of tensors, the bias / BatchNorm / activation / residual may be fused
into the convolution's single output store, and the tag ``'auto'`` lets the
engine choose the dataflow.
"""
from __future__ import annotations

import math
from typing import List, Optional, Union

import numpy as np
import torch
import torch.nn as nn

from . import functional as PF
from .functional import FusedEpilogue
from .kmap import KernelMap
from .sptensor import spTensor
from .utils import conv_info_decoder, conv_info_encoder, output_stride_compute

_ONES = conv_info_encoder([1, 1, 1])
_TAGS = ("D1", "D2", "auto")


def _triple(v, what):
    if isinstance(v, int):
        return [v, v, v]
    if isinstance(v, (list, tuple)) and len(v) == 3:
        return list(v)
    raise NotImplementedError(f"{what} must be an int or a list of three ints")


class conv3d(nn.Module):
    """Sparse 3-D convolution with the reference's constructor and parameters
    (script/spconv.py:15-106): ``kernel`` is [kv, C_in, C_out] (or [C_in, C_out] for a
    1x1x1 kernel), ``bias`` is [C_out] or None, both initialised U(+-1/sqrt(C_out*kv))."""

    def __init__(self, in_channels: int = 16, out_channels: int = 32, kernel_size: Union[int, List[int]] = 3,
                 stride: Union[int, List[int]] = 1, padding: Union[int, List[int]] = 0, bias: bool = False,
                 transposed: bool = False, tc_mode: bool = True) -> None:
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.transposed = transposed
        self.kernel_size = _triple(kernel_size, "kernel_size")
        self.kernel_size_code = conv_info_encoder(self.kernel_size)
        self.kernel_volume = int(np.prod(self.kernel_size, dtype=int))
        self.stride = _triple(stride, "stride")
        self.stride_code = conv_info_encoder(self.stride)
        self.padding = _triple(padding, "padding")
        self.padding_code = conv_info_encoder(self.padding)
        self.tensorcore = tc_mode
        shape = (self.kernel_volume, in_channels, out_channels) if self.kernel_volume > 1 else (in_channels, out_channels)
        self.kernel = nn.Parameter(torch.zeros(shape))
        self.bias = nn.Parameter(torch.zeros((out_channels,))) if bias else None
        self.reset_parameters()

    def extra_repr(self) -> str:
        s = f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}"
        if self.stride_code != _ONES:
            s += f", stride={self.stride}"
        if self.bias is None:
            s += ", bias=False"
        if self.transposed:
            s += ", transposed=True"
        return s

    def reset_parameters(self):
        bound = 1.0 / math.sqrt(self.out_channels * self.kernel_volume)
        self.kernel.data.uniform_(-bound, bound)
        if self.bias is not None:
            self.bias.data.uniform_(-bound, bound)
        PF.invalidate_packed(self.kernel)  # a write through .data does not advance the version the cache keys on

    def forward(self, input: spTensor, epilogue: Optional[FusedEpilogue] = None,
                out: Optional[torch.Tensor] = None) -> spTensor:
        """``out``: where the output features go, e.g. a column range of a wider matrix that a later
        layer reads whole (the result's ``feats`` is then that tensor)."""
        return conv_func(input=input, in_channel=self.in_channels, out_channel=self.out_channels, kernel=self.kernel,
                         kernel_size_code=self.kernel_size_code, stride_code=self.stride_code,
                         padding_code=self.padding_code, bias=self.bias, transposed=self.transposed,
                         tensorcore=self.tensorcore, epilogue=epilogue, out=out)


def _with_bias(epilogue: Optional[FusedEpilogue], bias) -> Optional[FusedEpilogue]:
    """Fold the layer bias into the epilogue: (acc + b)*s + t = acc*s + (b*s + t)."""
    if bias is None:
        return epilogue
    b = bias.detach().float()
    if epilogue is None:
        return FusedEpilogue(shift=b.contiguous())
    shift = b * epilogue.scale if epilogue.scale is not None else b
    if epilogue.shift is not None:
        shift = shift + epilogue.shift
    return epilogue.replace(shift=shift.contiguous())  # every other field (second operand, halo push) is kept


# Measured crossover of the two dataflows on B200 (submanifold 3x3x3, fp16, kernel-only, L2 flushed:
# `bench.py --workload selector`, summarised in profiles/selector_sweep.md): channel widths 16..256 x
# {indoor surfaces, LiDAR, fully dense block} x {about 25 k, 200 k rows}.  The fused output-stationary
# dataflow (D2) is faster in 35 of the 36 cells (by 1.0-16x; the explicit one moves 2*(C_in + C_out)*pairs
# extra elements through HBM).  The explicit dataflow (D1) wins where D2's per-tile weight staging
# dominates: wide layers on small, very sparse maps (256 -> 256 on 25 k rows with 1.2 pairs per row:
# 56 vs 82 us); at 96..128 channels on such maps the two tie (1.02-1.04).  Each entry: D1 when the
# layer is fp16, both widths >= c_min, the map has at most rows_max output rows and at most ppr_max pairs
# per row.
_D1_WINS = (dict(half=True, c_min=256, rows_max=40000, ppr_max=2.0),)


def _choose_dataflow(tag: str, in_channel: int, out_channel: int, pairs_per_row=None, n_rows: Optional[int] = None,
                     dtype=None) -> str:
    """'D1' / 'D2' are taken as given; 'auto' is the adaptive choice from channel widths, map size and
    sparsity (pairs per output row; a number, or a callable evaluated only when the cheaper conditions
    hold, since it costs a read-back of the pair count), looked up in the measured table ``_D1_WINS``.
    Without the facts an entry needs (no row count or sparsity given) the fused dataflow (D2) runs."""
    if tag != "auto":
        return tag
    for e in _D1_WINS:
        if (dtype == torch.float16) != e["half"] or min(in_channel, out_channel) < e["c_min"]:
            continue
        if n_rows is None or n_rows > e["rows_max"] or pairs_per_row is None:
            continue
        ppr = pairs_per_row() if callable(pairs_per_row) else pairs_per_row
        if ppr <= e["ppr_max"]:
            return "D1"
    return "D2"


def _run_conv(feats, w, kmap, transposed, ep, buffer, out=None):
    if kmap.dataflow == "D1":
        res = PF.conv_forward_d1(feats, w, kmap, transposed, ep, buffer)
        if out is not None:
            out.copy_(res)
            return out
        return res
    return PF.conv_forward(feats, w, kmap.csr(transposed=transposed), ep, out=out)


def _map_for(input, in_channel, out_channel, kernel_size_code, stride_code, padding_code):
    """The kernel map of a non-transposed layer applied to ``input``: fetched from ``input.kmaps`` or
    built and registered there (script/spconv.py:338-427).  Returns (map, output stride code,
    output coords_max, output coords_min)."""
    output_stride = output_stride_compute(stride_code, input.stride, 0)
    key = (kernel_size_code, input.stride, stride_code)
    kmap = input.kmaps.get(key)
    if kmap is None and input.planner is not None:
        kmap = input.planner.fetch(input, key, output_stride)
    subm = stride_code == _ONES
    coords_max = [input.coords_max[i] for i in range(3)]
    coords_min = [input.coords_min[i] for i in range(3)]
    ks = conv_info_decoder(kernel_size_code)
    stride = conv_info_decoder(stride_code)
    padding = conv_info_decoder(padding_code)
    if not subm:
        coords_max = [(input.coords_max[i] + 2 * padding[i] - (ks[i] - 1)) // stride[i] for i in range(3)]
    if kmap is None:
        tag = input.init_tag[0] if len(input.init_tag) else "end"
        if tag not in _TAGS:
            raise NotImplementedError(f"no dataflow tag left for a new kernel map (init_tag[0] = {tag!r})")
        kmap = KernelMap(input.coords, ks, stride, padding, coords_min, coords_max, subm)
        def pairs_per_row():  # incl. the centre offset of a submanifold map; one size read-back
            return (kmap.sizes()[0] + (kmap.n_in if subm else 0)) / max(kmap.n_out, 1)
        kmap.dataflow = _choose_dataflow(tag, in_channel, out_channel, pairs_per_row, kmap.n_out, input.feats.dtype)
        input.kmaps[key] = kmap
        input.cbook[output_stride] = kmap.out_coords
        if not (tag == "auto" and len(input.init_tag) == 1):
            input.init_tag = input.init_tag[1:]
    return kmap, output_stride, coords_max, coords_min


def _slab_submanifold(input, slabs, w, kernel_size_code, ep, out):
    """A submanifold layer on ONE RANK'S SLAB of a scene (``input.slabs``, a multigpu.SlabLevels): ``input`` holds
    the rows this rank owns at its level.  The level's halo rows are fetched from the neighbouring ranks, the map
    is built once per level and kernel size over [owned | halo] rows, and only the owned output rows are computed:
    they are the rows an undivided run returns for these voxels."""
    level = slabs.level_of(conv_info_decoder(input.stride))
    scene = slabs[level]
    ks = conv_info_decoder(kernel_size_code)
    if any(k % 2 == 0 for k in ks) or max(ks) // 2 > scene.radius:
        raise NotImplementedError("a submanifold layer on slabs needs odd kernel sizes within the slabs' halo radius")
    if input.feats.size(0) != scene.n_owned:
        raise ValueError("the tensor's rows are not the rows this rank owns at its level")
    key = ("slab", kernel_size_code, input.stride)
    entry = input.kmaps.get(key)
    if entry is None:
        tag = input.init_tag[0] if len(input.init_tag) else "end"
        if tag not in _TAGS:
            raise NotImplementedError(f"no dataflow tag left for a new kernel map (init_tag[0] = {tag!r})")
        kmap = KernelMap(scene.local_coords, ks, (1, 1, 1), (0, 0, 0), input.coords_min, input.coords_max, True)
        kmap.dataflow = "D2"  # (the restricted CSR below is the fused dataflow's)
        entry = input.kmaps[key] = (kmap, kmap.csr().restrict(scene.n_owned))
        if not (tag == "auto" and len(input.init_tag) == 1):
            input.init_tag = input.init_tag[1:]
    room = getattr(input, "halo_room", None)
    if scene.n_local == scene.n_owned:
        local = input.feats                   # nothing to fetch (one slab, or no voxel near a cut)
    elif (room is not None and room.size(0) == scene.n_local and room.dtype == input.feats.dtype
            and room.data_ptr() == input.feats.data_ptr() and room.size(1) == input.feats.size(1)):
        local = room                          # the layer that produced the rows left room for the halo behind them
    else:
        local = scene.alloc_local(input.feats.size(1), input.feats.dtype)
        local[: scene.n_owned] = input.feats
    slabs.exchange_into(level, local)
    return PF.conv_forward(local, w, entry[1], ep, out=out)


def _with_halo_room(slabs, stride_code: int, c_out: int, like: torch.Tensor, out):
    """Output storage of a layer on a slab tensor: ``out`` as given, else the first rows of an
    [owned | halo] matrix of the output's level, so that a submanifold layer that reads the result next
    receives its halo rows in place instead of copying the owned rows first.  Returns (out, matrix or None)."""
    if out is not None:
        return out, None
    scene = slabs[slabs.level_of(conv_info_decoder(stride_code))]
    room = torch.empty((scene.n_local, c_out), dtype=like.dtype, device=like.device)
    return room[: scene.n_owned], room


def conv_func(input, in_channel, out_channel, kernel, kernel_size_code, stride_code, padding_code, bias, transposed,
              tensorcore, epilogue: Optional[FusedEpilogue] = None, out: Optional[torch.Tensor] = None):
    """Run one sparse convolution on ``input`` and return the output ``spTensor`` (its features written
    into ``out`` when given)."""
    ep = _with_bias(epilogue, bias)
    planner = getattr(input, "planner", None)
    slabs = getattr(input, "slabs", None)  # one rank's slab of a scene: see _slab_submanifold
    w = kernel  # the Parameter itself: the packed tensor-core layout is cached on it

    if kernel_size_code == _ONES and stride_code == _ONES:
        out_feats = PF.linear_forward(input.feats, w if w.dim() == 2 else w[0], ep)
        if out is not None:
            out.copy_(out_feats)
            out_feats = out
        output = spTensor(coords=input.coords, feats=out_feats, buffer=input.buffer, batchsize=input.batchsize,
                          stride=input.stride, init_tag=input.init_tag, coords_max=input.coords_max,
                          coords_min=input.coords_min)

    elif transposed:
        output_stride = output_stride_compute(stride_code, input.stride, 1)
        kmap = input.kmaps.get((kernel_size_code, output_stride, stride_code))
        if kmap is None and planner is not None:
            kmap = planner.fetch(input, (kernel_size_code, output_stride, stride_code), None)
        if kmap is None:
            raise RuntimeError("transposed conv3d needs the kernel map of its matching strided conv3d "
                               "(same kernel size and stride) built earlier on this tensor's network")
        # the reference reads cbook[output_stride] and fails when no layer registered that
        # stride (script/spconv.py:309); the map itself remembers its fine side.
        out_coords = input.cbook.get(output_stride, kmap.in_coords)
        room = None
        if slabs is not None:
            out, room = _with_halo_room(slabs, output_stride, out_channel, input.feats, out)
        out_feats = _run_conv(input.feats, w, kmap, True, ep, input.buffer, out)
        output = spTensor(feats=out_feats, coords=out_coords, buffer=input.buffer, batchsize=input.batchsize,
                          stride=output_stride, init_tag=input.init_tag, coords_max=input.coords_max,
                          coords_min=input.coords_min)
        output.halo_room = room

    elif slabs is not None and stride_code == _ONES:
        out, room = _with_halo_room(slabs, input.stride, out_channel, input.feats, out)
        out_feats = _slab_submanifold(input, slabs, w, kernel_size_code, ep, out)
        output = spTensor(feats=out_feats, coords=input.coords, buffer=input.buffer, batchsize=input.batchsize,
                          stride=input.stride, init_tag=input.init_tag, coords_max=input.coords_max,
                          coords_min=input.coords_min)
        output.halo_room = room

    else:
        if slabs is not None and (kernel_size_code != stride_code or any(conv_info_decoder(padding_code))):
            raise NotImplementedError("a down-sampling layer on slabs needs kernel size == stride and no padding")
        kmap, output_stride, coords_max, coords_min = _map_for(input, in_channel, out_channel, kernel_size_code,
                                                               stride_code, padding_code)
        room = None
        if slabs is not None:
            out, room = _with_halo_room(slabs, output_stride, out_channel, input.feats, out)
        out_feats = _run_conv(input.feats, w, kmap, False, ep, input.buffer, out)
        output = spTensor(feats=out_feats, coords=kmap.out_coords, buffer=input.buffer, batchsize=input.batchsize,
                          stride=output_stride, init_tag=input.init_tag, coords_max=coords_max,
                          coords_min=coords_min)
        output.halo_room = room

    output.kmaps = input.kmaps
    output.cbook = input.cbook
    output.planner = planner
    output.slabs = slabs
    return output
