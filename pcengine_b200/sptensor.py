"""``spTensor``: the sparse-tensor container of the operator surface
(same fields and methods as the reference's script/sptensor.py:4-91)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


class spTensor:
    """feats [N,C], coords int32 [N,4] = (b,x,y,z), a stride code (94585 = (1,1,1)),
    the kernel-map cache ``kmaps`` and the coordinate book ``cbook`` shared along a
    network, the dataflow tag list ``init_tag`` and the coordinate bounds."""

    def __init__(self, feats: torch.Tensor, coords: torch.Tensor, buffer: Optional[torch.Tensor] = None,
                 coords_min: Optional[list] = None, coords_max: Optional[list] = None, batchsize: int = 1,
                 stride: int = 94585, init_tag: Optional[list] = None) -> None:
        self.feats = feats
        self.coords = coords
        self.stride = stride
        self.batchsize = batchsize
        self.buffer = buffer
        self.kmaps: Dict = {}
        self.cbook: Dict = {}
        self.planner = None       # the planner pass that builds this network pass's kernel maps (planner.MapPlan)
        self.coords_ready = None  # optional CUDA event after which `coords` is valid (read by MapPlan.begin)
        self.slabs = None         # multigpu.SlabLevels when the rows are one rank's slab of a scene (spconv.conv_func)
        self.halo_room = None     # slab tensors: the [owned | halo] matrix whose first rows `feats` are, if any
        self.init_tag = ["end"] if init_tag is None else init_tag
        self.coords_min = [0, 0, 0] if coords_min is None else coords_min
        if coords_max is None:
            coords_max = coords[:, 1:].max(dim=0).values.cpu().tolist() if coords.numel() else [0, 0, 0]
        self.coords_max = coords_max

    @property
    def F(self) -> torch.Tensor:
        return self.feats

    @F.setter
    def F(self, feats: torch.Tensor) -> None:
        self.feats = feats

    @property
    def C(self) -> torch.Tensor:
        return self.coords

    @C.setter
    def C(self, coords: torch.Tensor) -> None:
        self.coords = coords

    def cpu(self):
        self.coords = self.coords.cpu()
        self.feats = self.feats.cpu()
        return self

    def cuda(self):
        self.coords = self.coords.cuda()
        self.feats = self.feats.cuda()
        return self

    def detach(self):
        self.coords = self.coords.detach()
        self.feats = self.feats.detach()
        return self

    def to(self, device, non_blocking: bool = True):
        self.coords = self.coords.to(device, non_blocking=non_blocking)
        self.feats = self.feats.to(device, non_blocking=non_blocking)
        return self

    def build_buffer(self, cinfo: Dict, device):
        """Workspace for the explicit gather-GEMM-scatter dataflow, sized as
        script/sptensor.py:63-78 does (rows = nnz x {16|48|8|ks^3} for ks = 3|5|2|other)."""
        max_c_in = max(cinfo["in"])
        max_c_out = max(cinfo["out"])
        max_ks = max(cinfo["kernel"])
        nnz = self.coords.size(0)
        mult = {3: 16, 5: 48, 2: 8}.get(max_ks, max_ks ** 3)
        self.buffer = torch.zeros(((max_c_in + max_c_out) * nnz * mult,), dtype=torch.float, device=device)

    def _like(self, feats):
        out = spTensor(coords=self.coords, feats=feats, batchsize=self.batchsize, stride=self.stride,
                       init_tag=self.init_tag, buffer=self.buffer, coords_max=self.coords_max,
                       coords_min=self.coords_min)
        out.cbook = self.cbook
        out.kmaps = self.kmaps
        out.planner = self.planner
        out.slabs = self.slabs
        return out

    def __add__(self, other):
        return self._like(self.feats + other.feats)


SparseTensor = spTensor
