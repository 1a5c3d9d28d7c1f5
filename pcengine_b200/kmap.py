"""Host-side kernel-map object: owns the device arrays the C ABI fills and
derives the other forms lazily.  Mirrors what the reference keeps per
(kernel size, tensor stride, layer stride) in ``spTensor.kmaps``
(script/spconv.py:333,382-384,431-433)."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import lib

D1_CODE = 1186111  # backend/hash.cuh:7-9


def make_geom(ks, stride, pad, cmin, cmax, subm: bool) -> _lib.Geom:
    g = _lib.Geom()
    for i in range(3):
        g.ks[i] = int(ks[i])
        g.stride[i] = int(stride[i])
        g.pad[i] = int(pad[i])
        g.cmin[i] = int(cmin[i])
        g.cmax[i] = int(cmax[i])
    g.submanifold = 1 if subm else 0
    return g


def candidates_per_input(ks, stride) -> int:
    """Upper bound on the outputs one input voxel can feed in a strided conv."""
    n = 1
    for k, s in zip(ks, stride):
        n *= (k + s - 1) // s
    return n


# Rows per tile of the tile lists (128 or 256) when the caller does not say.
TILE_ROWS = 128


class NeighbourCSR:
    """mask [rows, ceil(kv/32)] uint32 (as int32 storage), rowptr [rows+1], nbr [cap].

    ``fill``: a callable returning (rowptr, nbr) for a CSR that arrives without them (a planned map
    whose tile lists were filled straight from the dense table); they are then built on first use."""

    __slots__ = ("mask", "_rowptr", "_nbr", "n_rows", "n_src", "kv", "_order", "_tiles", "_fill", "_pairs")

    def __init__(self, mask, rowptr, nbr, n_rows, n_src, kv=None, fill=None, pairs=None):
        self.mask, self._rowptr, self._nbr, self.n_rows, self.n_src = mask, rowptr, nbr, n_rows, n_src
        self.kv = kv
        self._order = None
        self._tiles = {}
        self._fill = fill
        self._pairs = pairs  # callable -> one-element device tensor, for a CSR without rowptr

    def pair_count(self) -> torch.Tensor:
        """Number of (row, offset) pairs as a NEW one-element device tensor (no read-back, and nothing that
        keeps the map's storage alive)."""
        if self._rowptr is None and self._pairs is not None:
            return self._pairs()
        return self.rowptr[-1:].clone()

    def _materialise(self):
        if self._rowptr is None and self._fill is not None:
            self._rowptr, self._nbr = self._fill()
            self._fill = None

    @property
    def rowptr(self):
        self._materialise()
        return self._rowptr

    @property
    def nbr(self):
        self._materialise()
        return self._nbr

    def restrict(self, n_rows: int) -> "NeighbourCSR":
        """The CSR of the first ``n_rows`` output rows only (same inputs, shared storage): what a
        slab of a scene uses to compute its owned rows and not the halo's."""
        if not 0 <= n_rows <= self.n_rows:
            raise ValueError("restrict: n_rows out of range")
        return NeighbourCSR(self.mask[:max(n_rows, 1)], self.rowptr[: n_rows + 1], self.nbr, n_rows, self.n_src, self.kv)

    def order(self):
        """Output rows sorted by indicator bitmask (int32 [n_rows], built once): the order in which
        the tensor-core kernel forms its 128-row tiles."""
        if self._order is None and self.n_rows == 0:
            self._order = torch.empty((0,), dtype=torch.int32, device=self.mask.device)
        if self._order is None and self.kv is not None:
            dev = self.mask.device
            out = torch.empty((self.n_rows,), dtype=torch.int32, device=dev)
            ws = _lib.workspace(64 * self.n_rows + (16 << 20), dev)
            _lib.check(lib.pce_csr_sort_rows(self.mask.data_ptr(), self.n_rows, self.kv, ws.data_ptr(), ws.numel(),
                                             out.data_ptr(), _lib.stream_ptr(dev)), "pce_csr_sort_rows")
            self._order = out
        return self._order

    def tiles(self, sort_rows: bool = True, tile_rows: int | None = None, identity: bool = False, slots: int = 1):
        """The map as tile lists (a ``_lib.TileLists`` struct of device pointers) for the
        tensor-core kernel; built once per CSR, ordering, tile height and ``identity`` (every tile
        ends with the stage where a second operand joins) and ``slots`` (offsets per stage: 64 / C_in
        for layers with 16 or 32 input channels), kept alive with it.  A request without ``identity``
        is also served by lists that have the stage: the kernel skips it."""
        tile_rows = int(tile_rows or TILE_ROWS)
        key = (bool(sort_rows), tile_rows, bool(identity), int(slots))
        hit = self._tiles.get(key)
        if hit is None and not identity:
            hit = self._tiles.get((bool(sort_rows), tile_rows, True, int(slots)))
        if hit is not None:
            # kept from an earlier call: once the kernels that built the lists have finished, a launch
            # may read the lists during its set-up (while the kernel before it is still finishing)
            if not hit[0].settled and (len(hit) < 6 or hit[5].query()):
                hit[0].settled = 1
            return hit[0]
        dev = self.mask.device
        n_tiles = (self.n_rows + tile_rows - 1) // tile_rows
        if sort_rows:
            order = self.order()
        else:
            order = torch.arange(self.n_rows, dtype=torch.int32, device=dev)
        cap = max(1, n_tiles * ((self.kv + slots - 1) // slots + (1 if identity else 0)))
        tile_ptr = torch.empty((n_tiles + 1,), dtype=torch.int32, device=dev)
        stage_kp = torch.empty((cap * slots,), dtype=torch.int32, device=dev)
        stage_nbr = torch.empty((cap * slots * tile_rows,), dtype=torch.int32, device=dev)
        ws = _lib.workspace(8 * (n_tiles + 1) + (1 << 20), dev)
        _lib.check(lib.pce_build_tile_lists(self.mask.data_ptr(), self.rowptr.data_ptr(), self.nbr.data_ptr(),
                                            order.data_ptr(), self.n_rows, self.kv, tile_rows, 1 if identity else 0, int(slots),
                                            ws.data_ptr(),
                                            ws.numel(),
                                            tile_ptr.data_ptr(), stage_kp.data_ptr(), stage_nbr.data_ptr(), cap,
                                            _lib.stream_ptr(dev)), "pce_build_tile_lists")
        st = _lib.TileLists(order.data_ptr(), tile_ptr.data_ptr(), stage_kp.data_ptr(), stage_nbr.data_ptr(),
                            tile_rows, 1 if identity else 0, int(slots), 0)
        built = torch.cuda.Event()
        built.record(torch.cuda.current_stream(dev))
        self._tiles[key] = (st, order, tile_ptr, stage_kp, stage_nbr, built)
        return st


class KernelMap:
    def __init__(self, in_coords: torch.Tensor, ks, stride, pad, cmin, cmax_out, subm: bool):
        _lib.require_cuda(in_coords, "coords")
        if in_coords.dtype != torch.int32 or in_coords.dim() != 2 or in_coords.size(1) != 4:
            raise ValueError("coords must be an int32 [N,4] tensor of (b,x,y,z)")
        in_coords = in_coords.contiguous()
        dev = in_coords.device
        self.device = dev
        self.ks, self.stride, self.pad = tuple(ks), tuple(stride), tuple(pad)
        self.subm = bool(subm)
        self.kv = int(ks[0] * ks[1] * ks[2])
        self.mid = (ks[0] - 1) // 2 * ks[1] * ks[2] + (ks[1] - 1) // 2 * ks[2] + (ks[2] - 1) // 2
        self.n_in = int(in_coords.size(0))
        self.in_coords = in_coords
        self.geom = make_geom(ks, stride, pad, cmin, cmax_out, subm)
        st = _lib.stream_ptr(dev)
        kv = self.kv
        if subm:
            self.out_coords = in_coords
            self.n_out = self.n_in
        else:
            cap = max(1, self.n_in * candidates_per_input(ks, stride))
            ws = _lib.workspace(lib.pce_map_workspace_bytes(self.n_in, kv, cap), dev)
            oc = torch.empty((cap, 4), dtype=torch.int32, device=dev)
            n_out = C.c_int32(0)
            _lib.check(lib.pce_downsample_coords(in_coords.data_ptr(), self.n_in, C.byref(self.geom), ws.data_ptr(),
                                                 ws.numel(), oc.data_ptr(), cap, C.byref(n_out), st),
                       "pce_downsample_coords")
            self.n_out = int(n_out.value)
            self.out_coords = oc[: self.n_out]
        self._built = False
        self._csr: dict = {}
        self._pairs = None
        self._d1 = None
        self._sizes = None
        self.dataflow = "D2"
        # A submanifold map with odd kernel sizes is its own transpose under kp -> kv-1-kp, so
        # the output-major table is read out of `map`; otherwise it is written separately.
        self.symmetric = self.subm and all(k % 2 == 1 for k in ks)
        self.build()

    def build(self) -> "KernelMap":
        """Hash the output coordinates, query every (input, offset) and scan the per-offset counts
        (idempotent), on PyTorch's current stream."""
        if self._built:
            return self
        dev, kv, in_coords = self.device, self.kv, self.in_coords
        st = _lib.stream_ptr(dev)
        ws = _lib.workspace(lib.pce_map_workspace_bytes(self.n_in, kv, self.n_out), dev)
        self.map = torch.empty((kv * self.n_in,), dtype=torch.int32, device=dev)
        # A submanifold map with odd kernel sizes is its own transpose under kp -> kv-1-kp, so
        # the output-major table is read out of `map`; otherwise it is written separately.
        self.map_out = None if self.symmetric else torch.empty((kv * max(self.n_out, 1),), dtype=torch.int32, device=dev)
        self.knnz = torch.empty((kv,), dtype=torch.int32, device=dev)
        self.kpos = torch.empty((kv + 1,), dtype=torch.int32, device=dev)
        self.qkpos = torch.empty((kv + 1,), dtype=torch.int32, device=dev)
        self.status = torch.zeros((1,), dtype=torch.int32, device=dev)
        _lib.check(lib.pce_map_build_d2(in_coords.data_ptr(), self.n_in, self.out_coords.data_ptr(), self.n_out,
                                        C.byref(self.geom), ws.data_ptr(), ws.numel(), _lib.ptr(self.map),
                                        self.knnz.data_ptr(), self.kpos.data_ptr(), self.qkpos.data_ptr(),
                                        _lib.ptr(self.map_out), self.status.data_ptr(), st), "pce_map_build_d2")
        self._built = True
        return self

    # -- sizes that live on the device -------------------------------------
    def sizes(self):
        """(pairs, qsum) read back once (one synchronisation), also validates the status word.
        The reference reads qkpos[-1] the same way (script/spconv.py:376,421)."""
        if self._sizes is None:
            self.build()
            host = torch.stack([self.kpos[-1], self.qkpos[-1], self.status[0]]).cpu()
            if int(host[2]) != 0:
                _lib.check(int(host[2]), "kernel map build")
            self._sizes = (int(host[0]), int(host[1]))
        return self._sizes

    # -- neighbour CSR + bitmask (what pce_conv_fwd consumes) ---------------
    def csr(self, transposed: bool = False) -> NeighbourCSR:
        key = bool(transposed)
        if key in self._csr:
            return self._csr[key]
        self.build()
        dev, kv = self.device, self.kv
        st = _lib.stream_ptr(dev)
        ident = self.mid if self.subm else -1
        if self.symmetric:
            # the table read with kp reversed is the output-major one; under `transposed`
            # (roles swapped) the table itself is.
            table, n_rows, n_src, reverse = self.map, self.n_out, self.n_in, (0 if transposed else 1)
        elif transposed:
            table, n_rows, n_src, reverse = self.map, self.n_in, self.n_out, 0
        else:
            table, n_rows, n_src, reverse = self.map_out, self.n_out, self.n_in, 0
        words = (kv + 31) // 32
        cap = max(1, kv * min(self.n_in, self.n_out) if not self.subm else kv * self.n_in)
        if self._sizes is not None:
            cap = max(1, self._sizes[0] + (self.n_in if self.subm else 0))
        mask = torch.empty((max(n_rows, 1), words), dtype=torch.int32, device=dev)
        rowptr = torch.empty((n_rows + 1,), dtype=torch.int32, device=dev)
        nbr = torch.empty((cap,), dtype=torch.int32, device=dev)
        ws = _lib.workspace(8 * (n_rows + 1) + (8 << 20), dev)
        _lib.check(lib.pce_csr_from_dense(_lib.ptr(table), kv, n_rows, reverse, ident, ws.data_ptr(), ws.numel(),
                                          mask.data_ptr(), rowptr.data_ptr(), nbr.data_ptr(), cap, st),
                   "pce_csr_from_dense")
        out = NeighbourCSR(mask, rowptr, nbr, n_rows, n_src, kv)
        self._csr[key] = out
        return out

    # -- reference forms -----------------------------------------------------
    def pairs(self):
        """(imap, omap) int32 [P], ordered by (kp, in): script/spconv.py:370-372."""
        if self._pairs is None:
            p, _ = self.sizes()
            dev = self.device
            imap = torch.empty((p,), dtype=torch.int32, device=dev)
            omap = torch.empty((p,), dtype=torch.int32, device=dev)
            ws = _lib.workspace(8 * self.kv * max(self.n_in, 1) + (16 << 20), dev)
            _lib.check(lib.pce_map_pairs(_lib.ptr(self.map), self.kv, self.n_in, ws.data_ptr(), ws.numel(),
                                         imap.data_ptr(), omap.data_ptr(), p, _lib.stream_ptr(dev)), "pce_map_pairs")
            self._pairs = (imap, omap)
        return self._pairs

    def d1(self):
        """(imap_coded [P], icsr [n_in+1], omap_coded [P], ocsr [n_out+1]): the CSR-coded
        gather/scatter map of backend/hash.cu:20-255 with canonical positions."""
        if self._d1 is None:
            p, _ = self.sizes()
            dev = self.device
            imap_c = torch.empty((max(p, 1),), dtype=torch.int32, device=dev)
            omap_c = torch.empty((max(p, 1),), dtype=torch.int32, device=dev)
            icsr = torch.empty((self.n_in + 1,), dtype=torch.int32, device=dev)
            ocsr = torch.empty((self.n_out + 1,), dtype=torch.int32, device=dev)
            ws = _lib.workspace(8 * self.kv * max(self.n_in, 1) + 8 * (max(self.n_in, self.n_out) + 1) + (16 << 20), dev)
            _lib.check(lib.pce_map_build_d1(_lib.ptr(self.map), _lib.ptr(self.map_out), self.kv, self.n_in, self.n_out,
                                            1 if self.symmetric else 0, self.kpos.data_ptr(), ws.data_ptr(), ws.numel(),
                                            imap_c.data_ptr(), icsr.data_ptr(), omap_c.data_ptr(), ocsr.data_ptr(),
                                            _lib.stream_ptr(dev)), "pce_map_build_d1")
            self._d1 = (imap_c[:p], icsr, omap_c[:p], ocsr)
        return self._d1


def csr_from_pairs(rows: torch.Tensor, nbrs: torch.Tensor, kpos: torch.Tensor, kv: int, n_rows: int,
                   n_src: int, identity_kp: int = -1) -> NeighbourCSR:
    """Neighbour CSR from (kp, in)-ordered pair lists (the only map data the reference's
    conv_fwd_d2_cuda receives, backend/spconv.h:28-40)."""
    dev = rows.device
    n_pairs = int(rows.numel())
    words = (kv + 31) // 32
    cap = max(1, n_pairs + (n_rows if identity_kp >= 0 else 0))
    mask = torch.empty((max(n_rows, 1), words), dtype=torch.int32, device=dev)
    rowptr = torch.empty((n_rows + 1,), dtype=torch.int32, device=dev)
    nbr = torch.empty((cap,), dtype=torch.int32, device=dev)
    ws = _lib.workspace(lib.pce_csr_from_pairs_workspace_bytes(n_pairs, n_rows), dev)
    _lib.check(lib.pce_csr_from_pairs(_lib.ptr(rows), _lib.ptr(nbrs), kpos.data_ptr(), kv, n_pairs, n_rows,
                                      identity_kp, ws.data_ptr(), ws.numel(), mask.data_ptr(), rowptr.data_ptr(),
                                      nbr.data_ptr(), cap, _lib.stream_ptr(dev)), "pce_csr_from_pairs")
    return NeighbourCSR(mask, rowptr, nbr, n_rows, n_src, kv)
