"""Host utilities of the operator surface (counterparts of script/utils.py):
geometry codes, stride composition, ``fapply``/``cat``, voxel quantisation,
collation and the dataflow heuristic."""
from __future__ import annotations

from itertools import repeat
from typing import Any, Callable, Dict, List, Tuple, Union

import numpy as np
import torch

from .sptensor import spTensor


def conv_info_encoder(info: List[int]) -> int:
    """(x,y,z) -> 94273*x + 311*y + z (script/utils.py:233-234)."""
    return 94273 * info[0] + 311 * info[1] + info[2]


def conv_info_decoder(code: int) -> Tuple[int, int, int]:
    """Inverse of :func:`conv_info_encoder` (script/utils.py:237-242)."""
    x = code // 94273
    y = (code - x * 94273) // 311
    z = code - x * 94273 - y * 311
    return (x, y, z)


def output_stride_compute(l_stride_code: int, t_stride_code: int, transposed: bool = False) -> int:
    """Tensor stride after a layer: multiplied by the layer stride, or divided by it for a
    transposed layer (script/utils.py:116-138)."""
    l, t = conv_info_decoder(l_stride_code), conv_info_decoder(t_stride_code)
    s = [t[i] // l[i] for i in range(3)] if transposed else [t[i] * l[i] for i in range(3)]
    return conv_info_encoder(s)


def fapply(input: spTensor, fn: Callable[..., torch.Tensor], *args, **kwargs) -> spTensor:
    """Apply ``fn`` to the feature rows, keep everything else (script/utils.py:141-149)."""
    return input._like(fn(input.feats, *args, **kwargs))


def cat(inputs: List[spTensor]) -> spTensor:
    """Channel concatenation of tensors on the same coordinates (script/utils.py:152-164)."""
    return inputs[0]._like(torch.cat([x.feats for x in inputs], dim=1))


def ravel_hash(x: np.ndarray) -> np.ndarray:
    """Row-major linear index of integer rows inside their bounding box (script/utils.py:18-31)."""
    if x.ndim != 2:
        raise ValueError(f"expected [N,D] integer rows, got {x.shape}")
    lo = x.min(axis=0)
    extent = (x.max(axis=0) - lo + 1).astype(np.int64)
    return np.ravel_multi_index(tuple((x - lo).T.astype(np.int64)), tuple(extent)).astype(np.uint64)


def sparse_quantize(coords, voxel_size: Union[float, Tuple[float, ...]] = 1, *, return_index: bool = False,
                    return_inverse: bool = False):
    """floor(coords / voxel) and keep one point per voxel (script/utils.py:34-55).  A CUDA tensor of
    points is voxelised on the device (pce_quantize_unique) and CUDA tensors come back: int32 [M,3]
    voxels in the same order as the host path, int64 ``indices`` / ``inverse``."""
    if isinstance(voxel_size, (float, int)):
        voxel_size = tuple(repeat(voxel_size, 3))
    assert isinstance(voxel_size, tuple) and len(voxel_size) == 3
    if isinstance(coords, torch.Tensor) and coords.is_cuda:
        return _sparse_quantize_cuda(coords, voxel_size, return_index, return_inverse)
    coords = np.floor(coords / np.array(voxel_size)).astype(np.int32)
    _, indices, inverse = np.unique(ravel_hash(coords), return_index=True, return_inverse=True)
    outputs = [coords[indices]]
    if return_index:
        outputs.append(indices)
    if return_inverse:
        outputs.append(inverse)
    return outputs[0] if len(outputs) == 1 else outputs


def _sparse_quantize_cuda(points: torch.Tensor, voxel_size, return_index: bool, return_inverse: bool):
    import ctypes as C

    from . import _lib
    from ._lib import lib
    if points.dim() != 2 or points.size(1) != 3:
        raise ValueError("points must be [N,3]")
    if points.dtype == torch.float64:
        raise NotImplementedError("device voxelisation takes float32 points (the host path handles float64)")
    pts = points.detach().to(torch.float32).contiguous()
    n, dev = pts.size(0), pts.device
    out = torch.empty((max(n, 1), 4), dtype=torch.int32, device=dev)
    index = torch.empty((max(n, 1),), dtype=torch.int32, device=dev) if return_index else None
    inverse = torch.empty((max(n, 1),), dtype=torch.int32, device=dev) if return_inverse else None
    ws = _lib.workspace(lib.pce_quantize_workspace_bytes(n), dev)
    voxel = (C.c_float * 3)(*[float(v) for v in voxel_size])
    m = C.c_int32(0)
    _lib.check(lib.pce_quantize_unique(pts.data_ptr(), n, voxel, 0, ws.data_ptr(), ws.numel(), out.data_ptr(),
                                       _lib.ptr(index), _lib.ptr(inverse), C.byref(m), _lib.stream_ptr(dev)),
               "pce_quantize_unique")
    outputs = [out[: m.value, 1:].contiguous()]
    if return_index:
        outputs.append(index[: m.value].long())
    if return_inverse:
        outputs.append(inverse[:n].long())
    return outputs[0] if len(outputs) == 1 else outputs


def build_conv_buffer(channel_list: Dict, nnz: int, data_type, device):
    """Gather/scatter workspace sized as script/utils.py:58-79."""
    max_ks = max(channel_list["kernel"])
    mult = {3: 16, 5: 48, 2: 8}.get(max_ks, max_ks ** 3 - 1)
    size = (max(channel_list["in"]) + max(channel_list["out"])) * nnz * mult
    return torch.zeros((size,), dtype=data_type, device=device)


def init_layer_scheduler(conv_info: Dict) -> str:
    """'whole' (build the gather/scatter map) when a layer at the input resolution has more
    than 32 channels on either side, else 'simple' (fetch on demand): the rule of
    script/utils.py:82-113, with its transposed-layer branch made reachable (the
    reference tests ``any(stride) < 1``, which is never true)."""
    stride, cin, cout = conv_info["stride"], conv_info["in"], conv_info["out"]
    for i, s in enumerate(stride):
        if s > 1:
            break
        if cin[i] > 32 or cout[i] > 32:
            return "whole"
    if any(s < 1 for s in stride):
        mul = 1.0
        for i, s in enumerate(stride):
            mul *= s
            if mul == 1 and (cin[i] > 32 or cout[i] > 32):
                return "whole"
    return "simple"


def sparse_collate(inputs: List[spTensor], init_tag=None) -> spTensor:
    """Stack samples into one batch, prepending the sample index to the coordinates
    (script/utils.py:167-196).  Unlike the reference the result carries a usable
    ``init_tag`` (the first sample's, or the one given) so a conv can run on it."""
    coords, feats = [], []
    stride = inputs[0].stride
    k = -1
    for k, x in enumerate(inputs):
        if isinstance(x.coords, np.ndarray):
            x.coords = torch.tensor(x.coords)
        if isinstance(x.feats, np.ndarray):
            x.feats = torch.tensor(x.feats)
        assert isinstance(x.coords, torch.Tensor), type(x.coords)
        assert isinstance(x.feats, torch.Tensor), type(x.feats)
        assert x.stride == stride, (x.stride, stride)
        c = x.coords[:, -3:].to(torch.int32)
        batch = torch.full((c.shape[0], 1), k, device=c.device, dtype=torch.int32)
        coords.append(torch.cat((batch, c), dim=1))
        feats.append(x.feats)
    coords = torch.cat(coords, dim=0)
    feats = torch.cat(feats, dim=0)
    coords_max = torch.max(coords[:, 1:], dim=0).values.cpu().numpy().tolist()
    tag = init_tag if init_tag is not None else inputs[0].init_tag
    return spTensor(coords=coords, feats=feats, stride=stride, batchsize=k + 1, buffer=None,
                    coords_min=[0, 0, 0], coords_max=coords_max, init_tag=tag)


def sparse_collate_fn(inputs: List[Any]) -> Any:
    """Dictionary-aware collate for data loaders (script/utils.py:199-217): nested dicts
    recurse, arrays/tensors concatenate on dim 0, spTensors go through sparse_collate,
    anything else is returned as a list."""
    if not isinstance(inputs[0], dict):
        return inputs

    def merge(values):
        head = values[0]
        if isinstance(head, dict):
            return sparse_collate_fn(values)
        if isinstance(head, spTensor):
            return sparse_collate(values)
        if isinstance(head, np.ndarray):
            return torch.cat([torch.as_tensor(v) for v in values], dim=0)
        if isinstance(head, torch.Tensor):
            return torch.cat(values, dim=0)
        return list(values)

    return {name: merge([sample[name] for sample in inputs]) for name in inputs[0]}


def make_ntuple(x, ndim: int) -> Tuple[int, ...]:
    """int | list | tuple | tensor -> tuple of ``ndim`` ints (script/utils.py:220-230)."""
    if isinstance(x, int):
        x = tuple(repeat(x, ndim))
    elif isinstance(x, list):
        x = tuple(x)
    elif isinstance(x, torch.Tensor):
        x = tuple(x.view(-1).cpu().numpy().tolist())
    assert isinstance(x, tuple) and len(x) == ndim, x
    return x
