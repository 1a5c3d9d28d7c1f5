"""``MapPlan``: every kernel map of a network pass, built ahead of the feature kernels by the
library's planning thread on a CUDA stream of its own (include/pce_b200.h, "kernel-map planner").

The reference builds each map inside the first convolution that needs it
(script/spconv.py:338-427).  Here a network declares its convolutions once::

    plan = MapPlan([(3, 1, False, 4, 32), (2, 2, False, 32, 32), (3, 1, False, 32, 64), (2, 2, True, 64, 32)])
    plan.begin(x)        # x: the input spTensor of a pass; returns at once
    y = net(x)           # conv_func finds the planned maps instead of building them

and the maps land in ``x.kmaps`` / ``x.cbook`` as the lazy path would leave them (same entry
points, bit-identical arrays), except that their storage belongs to the pass and is recycled
once no tensor of the pass refers to it any more.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import torch

from . import _lib
from . import functional as PF
from ._lib import lib
from .kmap import KernelMap, NeighbourCSR, make_geom
from .spconv import _ONES, _triple
from .utils import conv_info_decoder, conv_info_encoder, output_stride_compute


class _ArrayInterface:
    """CUDA array interface record of memory owned by ``keep``."""

    __slots__ = ("__cuda_array_interface__", "keep")

    def __init__(self, record, keep):
        self.__cuda_array_interface__, self.keep = record, keep


class _DevArray:
    """int32 device memory owned by a planner pass: enough of a tensor for the code that only
    needs the address (``data_ptr`` / ``device``), a real tensor on demand (zero-copy, through the
    CUDA array interface) for code that reads values."""

    __slots__ = ("ptr", "shape", "device", "_keep", "_tensor")

    def __init__(self, ptr: int, shape, device, keep):
        self.ptr, self.shape, self.device, self._keep, self._tensor = int(ptr or 0), tuple(shape), device, keep, None

    def data_ptr(self) -> int:
        return self.ptr

    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            if self.numel() == 0 or self.ptr == 0:
                self._tensor = torch.empty(self.shape, dtype=torch.int32, device=self.device)
            else:
                # the tensor keeps `view` (and through it the pass) alive, not this object: no cycle
                view = _ArrayInterface({"shape": self.shape, "typestr": "<i4", "data": (self.ptr, False), "version": 3,
                                        "strides": None}, self._keep)
                self._tensor = torch.as_tensor(view, device=self.device)
        return self._tensor

    def __getitem__(self, i):
        return self.tensor()[i]

    def cpu(self):
        return self.tensor().cpu()


class _PassHandle:
    """Owns a ``pce_pass``; releases it to the plan when the last user goes away."""

    def __init__(self, plan, handle, device, stream):
        self.plan, self.handle, self.device = plan, handle, device
        self.stream = stream  # the stream the maps are read on: the one of the latest fetch

    def __del__(self):
        h, self.handle = self.handle, None
        if h and self.plan.handle:
            # a failure (say, the stream no longer exists) leaves the pass unrecycled, which is safe
            lib.pce_pass_release(h, self.stream)


def _csr_filler(table: int, kv: int, n_rows: int, reverse_kp: int, identity_kp: int, cap: int, device, keep):
    """rowptr / nbr of one direction of a planned map, from its dense table (pce_csr_from_dense)."""
    def fill():
        words = (kv + 31) // 32
        mask = torch.empty((max(n_rows, 1), words), dtype=torch.int32, device=device)
        rowptr = torch.empty((n_rows + 1,), dtype=torch.int32, device=device)
        nbr = torch.empty((max(cap, 1),), dtype=torch.int32, device=device)
        ws = _lib.workspace(8 * (n_rows + 1) + (8 << 20), device)
        _lib.check(lib.pce_csr_from_dense(table, kv, n_rows, reverse_kp, identity_kp, ws.data_ptr(), ws.numel(),
                                          mask.data_ptr(), rowptr.data_ptr(), nbr.data_ptr(), max(cap, 1),
                                          _lib.stream_ptr(device)), "pce_csr_from_dense")
        return rowptr, nbr

    fill.keep = keep  # the table lives in the pass's arena: the pass stays alive as long as this does
    return fill


def _pair_counter(knnz, identity_rows: int):
    """Pairs of one direction of a map = the sum of its knnz, plus one per row where the rows name themselves
    at the identity offset (whose knnz is 0)."""
    def count():
        total = knnz.tensor().sum(0, keepdim=True, dtype=torch.int32)
        return total.add_(identity_rows) if identity_rows else total
    return count


class PlannedKernelMap(KernelMap):
    """A :class:`KernelMap` whose arrays were produced by the planner."""

    def __init__(self, out: _lib.PlannedMap, spec: dict, in_coords: torch.Tensor, cmin, keep, device):
        self.device = device
        self.ks, self.stride, self.pad = spec["ks"], spec["stride"], spec["pad"]
        self.subm = spec["subm"]
        ks = self.ks
        self.kv = int(out.kv)
        self.mid = (ks[0] - 1) // 2 * ks[1] * ks[2] + (ks[1] - 1) // 2 * ks[2] + (ks[2] - 1) // 2
        self.n_in, self.n_out = int(out.n_in), int(out.n_out)
        self.in_coords = in_coords
        self.geom = make_geom(ks, self.stride, self.pad, cmin, list(out.cmax_out), self.subm)
        self.out_coords = in_coords if self.subm else _DevArray(out.out_coords, (self.n_out, 4), device, keep).tensor()
        kv = self.kv
        self.map = _DevArray(out.map, (kv * self.n_in,), device, keep)
        self.symmetric = bool(out.symmetric)
        self.map_out = None if self.symmetric else _DevArray(out.map_out, (kv * max(self.n_out, 1),), device, keep)
        self.knnz = _DevArray(out.knnz, (kv,), device, keep)
        self.kpos = _DevArray(out.kpos, (kv + 1,), device, keep)
        self.qkpos = _DevArray(out.qkpos, (kv + 1,), device, keep)
        self.status = _DevArray(out.status, (1,), device, keep)
        self._built = True
        self._csr = {}
        self._pairs = self._d1 = self._sizes = None
        self.dataflow = "D2"
        for transposed, has, c in ((False, out.has_fwd, out.fwd), (True, out.has_tr, out.tr)):
            if not has:
                continue
            words = (kv + 31) // 32
            mask = _DevArray(c.mask, (max(c.n_rows, 1), words), device, keep)
            if c.rowptr:
                csr = NeighbourCSR(mask, _DevArray(c.rowptr, (c.n_rows + 1,), device, keep),
                                   _DevArray(c.nbr, (c.nbr_cap,), device, keep), int(c.n_rows), int(c.n_src), kv)
            else:
                # planned without its neighbour CSR (only tile lists were needed): built on first use
                csr = NeighbourCSR(mask, None, None, int(c.n_rows), int(c.n_src), kv,
                                   fill=_csr_filler(int(c.table), kv, int(c.n_rows), int(c.reverse_kp), int(c.identity_kp),
                                                    int(c.nbr_cap), device, keep),
                                   pairs=_pair_counter(self.knnz, int(c.n_rows) if c.identity_kp >= 0 else 0))
            for i in range(c.n_lists):
                t = c.lists[i]
                slots = max(int(t.slots), 1)
                lists = _lib.TileLists(t.order, t.tile_ptr, t.stage_kp, t.stage_nbr, t.tile_rows, t.identity_stage, slots,
                                       t.settled)
                n_tiles = (csr.n_rows + t.tile_rows - 1) // t.tile_rows
                csr._order = _DevArray(t.order, (csr.n_rows,), device, keep)
                entries = n_tiles * ((kv + slots - 1) // slots + int(t.identity_stage)) * slots
                csr._tiles[(True, int(t.tile_rows), bool(t.identity_stage), slots)] = (
                    lists, csr._order, _DevArray(t.tile_ptr, (n_tiles + 1,), device, keep),
                    _DevArray(t.stage_kp, (entries,), device, keep),
                    _DevArray(t.stage_nbr, (entries * t.tile_rows,), device, keep))
            self._csr[transposed] = csr


class PlannedPass:
    """What ``spTensor.planner`` holds during a planned pass."""

    def __init__(self, plan: "MapPlan", handle: _PassHandle, x):
        self.plan, self._handle = plan, handle
        self.device = x.coords.device
        self.cmin = list(x.coords_min)
        self.level_coords: List[Optional[torch.Tensor]] = [x.coords] + [None] * plan.n_levels

    def fetch(self, input, key, output_stride):
        """The planned map under ``key`` (host-waits until its kernels are queued and makes the
        current stream wait for them), registered in ``input.kmaps`` / ``input.cbook``; None when
        the key is not part of the plan."""
        idx = self.plan.index.get(key)
        if idx is None:
            return None
        spec = self.plan.specs[idx]
        out = _lib.PlannedMap()
        stream = _lib.stream_ptr(self.device)
        _lib.check(lib.pce_pass_map(self._handle.handle, idx, stream, C.byref(out)), "pce_pass_map")
        self._handle.stream = stream
        in_coords = self.level_coords[spec["in_level"]]
        if in_coords is None:
            in_coords = _DevArray(out.in_coords, (out.n_in, 4), self.device, self._handle).tensor()
            self.level_coords[spec["in_level"]] = in_coords
        kmap = PlannedKernelMap(out, spec, in_coords, self.cmin, self._handle, self.device)
        if not spec["subm"]:
            self.level_coords[spec["out_level"]] = kmap.out_coords
        input.kmaps[key] = kmap
        input.cbook[spec["out_stride"]] = kmap.out_coords
        return kmap


class MapPlan:
    """The kernel maps of a network, declared once.

    ``layers``: the convolutions in forward order as ``(kernel_size, stride, transposed, C_in,
    C_out)`` (ints or triples, padding 0; 1x1x1 stride-1 layers may be listed and are skipped).
    ``stride``: the stride code of the tensors the network takes (94585 = (1,1,1))."""

    def __init__(self, layers, stride: int = 94585, dtype=torch.float16):
        self.dtype = dtype
        self.in_stride = stride
        self.index: Dict[tuple, int] = {}
        self.specs: List[dict] = []
        level_of = {stride: 0}
        cur = stride
        for kernel_size, layer_stride, transposed, c_in, c_out in layers:
            ks, st = _triple(kernel_size, "kernel_size"), _triple(layer_stride, "stride")
            ks_code, st_code = conv_info_encoder(ks), conv_info_encoder(st)
            if ks_code == _ONES and st_code == _ONES:
                continue
            out_stride = output_stride_compute(st_code, cur, 1 if transposed else 0)
            key = (ks_code, out_stride if transposed else cur, st_code)
            if key not in self.index:
                if transposed:
                    raise RuntimeError("MapPlan: a transposed layer precedes its matching strided layer")
                subm = st_code == _ONES
                spec = dict(ks=tuple(ks), stride=tuple(st), pad=(0, 0, 0), subm=subm, in_level=level_of[cur],
                            out_stride=out_stride, fwd=[], tr=[])
                if not subm:
                    if out_stride in level_of:
                        raise NotImplementedError("MapPlan: two strided layers produce the same tensor stride")
                    level_of[out_stride] = len(level_of)
                spec["out_level"] = level_of[out_stride]
                self.index[key] = len(self.specs)
                self.specs.append(spec)
            spec = self.specs[self.index[key]]
            uses = spec["tr" if transposed else "fwd"]
            use = (PF._ceil16(c_out), PF._ceil16(c_in))
            if use not in uses and len(uses) < _lib.PLAN_MAX_USES - 1:
                uses.append(use)
            cur = out_stride
        if not self.specs:
            raise ValueError("MapPlan: no layer needs a kernel map")
        self.n_levels = len(level_of) - 1
        self.handles: Dict[int, int] = {}
        self.gates: Dict = {}  # per device: a stream that carries nothing but coordinate-ready events
        self.handle = True  # cleared when the plan is closed

    def _c_specs(self):
        arr = (_lib.PlanMapSpec * len(self.specs))()
        tensor_cores = self.dtype == torch.float16
        for s, c in zip(self.specs, arr):
            for d in range(3):
                c.ks[d], c.stride[d], c.pad[d] = s["ks"][d], s["stride"][d], s["pad"][d]
            c.in_level, c.submanifold = s["in_level"], 1 if s["subm"] else 0
            c.want_fwd, c.want_tr = (1 if s["fwd"] else 0), (1 if s["tr"] else 0)
            for name in ("fwd", "tr"):
                dst_out, dst_in = (c.c_out_fwd, c.c_in_fwd) if name == "fwd" else (c.c_out_tr, c.c_in_tr)
                widths = [u for u in s[name] if tensor_cores and u[0] <= 256]
                for i, (w_out, w_in) in enumerate(widths):
                    dst_out[i], dst_in[i] = w_out, (w_in if PF.PACK_OFFSETS else 0)
        return arr

    def _handle_for(self, device) -> int:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        h = self.handles.get(idx)
        if h is None:
            out = C.c_void_p()
            with torch.cuda.device(idx):
                arr = self._c_specs()
                _lib.check(lib.pce_plan_create(arr, len(self.specs), C.byref(out)), "pce_plan_create")
            h = self.handles[idx] = out.value
        return h

    def begin(self, x) -> bool:
        """Start building the maps for the pass whose input tensor is ``x`` and attach the pass to
        it; conv_func picks the maps up from there.  The planner waits for the producer of the
        coordinates only: everything queued so far on the current stream, or, when the tensor
        carries a CUDA event in ``x.coords_ready``, just that event, which lets the maps of the
        next pass be built while the current pass still computes.  Returns False (and leaves ``x``
        on the lazy path) when the tensor does not fit the plan (other stride, maps already
        present, an override of the tile policy in force, an empty tensor) or when eight earlier
        passes of this plan are still referenced (their maps kept alive by the caller)."""
        coords = x.coords
        if (not self.handle or not coords.is_cuda or coords.size(0) == 0 or x.stride != self.in_stride or x.kmaps
                or PF.TILE_ROWS is not None or not PF.SORT_ROWS or coords.dtype != torch.int32
                or not coords.is_contiguous()):
            return False
        dev = coords.device
        h = self._handle_for(dev)
        cmin = (C.c_int32 * 3)(*[int(v) for v in x.coords_min])
        cmax = (C.c_int32 * 3)(*[int(v) for v in x.coords_max])
        out = C.c_void_p()
        with torch.cuda.device(dev):
            stream = _lib.stream_ptr(dev)
            ready = getattr(x, "coords_ready", None)
            if ready is not None:
                gate = self.gates.get(dev)
                if gate is None:
                    gate = self.gates[dev] = torch.cuda.Stream(dev)
                gate.wait_event(ready)
                stream = gate.cuda_stream
            status = lib.pce_plan_begin(h, coords.data_ptr(), coords.size(0), cmin, cmax, stream, C.byref(out))
            if status == _lib.PCE_ERR_CAPACITY:  # too many passes are still referenced: this one builds lazily
                return False
            _lib.check(status, "pce_plan_begin")
        x.planner = PlannedPass(self, _PassHandle(self, out.value, dev, _lib.stream_ptr(dev)), x)
        return True

    def close(self) -> None:
        """Stop the planning threads and free their storage (passes must be finished)."""
        self.handle = False
        for h in self.handles.values():
            lib.pce_plan_destroy(h)
        self.handles = {}

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
