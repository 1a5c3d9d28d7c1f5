"""Multi-GPU helpers for the two ways the sparse-convolution path shards (the reference has no
multi-GPU support at all, so nothing here mirrors reference code):

* scan-parallel: independent scans go to different ranks; nothing is exchanged on the data path
  (``scans_for_rank``, ``max_over_ranks`` for device-side timing);
* slab-parallel: ONE large scene is cut along x into slabs with balanced voxel counts; every rank
  owns the outputs of its slab and needs the inputs within the kernel radius of its cut planes.
  Coordinates of that halo are exchanged once, features before every layer, either with
  neighbour-only point-to-point messages (``torch.distributed`` isend/irecv: NCCL over NVLink between
  GPUs, gloo in the CPU tests) or, between GPUs, by the convolution kernel itself storing its boundary
  rows into the neighbours' halo rows (``PeerPush``).  Halo rows land in the rank's own memory before
  any kernel reads them.  A network with down- and up-sampling layers runs on a ``SlabLevels``: one
  slab decomposition per coordinate level, with cut planes that are multiples of the coarsest level's
  stride, so that a down-sampling layer with kernel size == stride (and its transposed layer) reads
  and writes owned rows only and exchanges nothing; the submanifold layers of every level exchange
  that level's halo.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist


def scans_for_rank(n_scans: int, rank: int, world: int) -> List[int]:
    """Contiguous, balanced share of ``n_scans`` independent scans for ``rank``."""
    base, extra = divmod(n_scans, world)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def max_over_ranks(value: float, device=None) -> float:
    """Maximum of a host float over all ranks (the step time of a multi-GPU run)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def slab_cuts(x: np.ndarray, world: int, radius: int) -> List[int]:
    """``world + 1`` cut planes along x (cuts[g] <= x < cuts[g+1] is owned by rank g) that balance the
    voxel counts; every slab is at least ``radius`` wide so a halo never reaches past a neighbour."""
    x = np.asarray(x, dtype=np.int64)
    lo, hi = int(x.min()), int(x.max()) + 1
    if world == 1:
        return [lo, hi]
    hist = np.bincount(x - lo, minlength=hi - lo)
    cum = np.concatenate([[0], np.cumsum(hist)])
    cuts = [lo]
    for g in range(1, world):
        target = cum[-1] * g / world
        c = lo + int(np.searchsorted(cum, target))
        c = max(c, cuts[-1] + max(radius, 1))
        cuts.append(c)
    cuts.append(hi)
    for g in range(world):
        if cuts[g + 1] - cuts[g] < max(radius, 1):
            raise ValueError("scene too thin along x for this many slabs and this kernel radius")
    return cuts


def aligned_slab_cuts(x: np.ndarray, world: int, radius: int, align: int) -> List[int]:
    """``slab_cuts`` with every plane a multiple of ``align`` (the product of the strides down to the
    coarsest level that is cut): a coarse voxel's children then all belong to one rank on every level.
    Every slab is at least ``radius * align`` wide, so the coarsest level's halo (``radius`` coarse
    voxels) still lies inside the neighbouring slab.  Coordinates must be non-negative."""
    x = np.asarray(x, dtype=np.int64)
    if align < 1:
        raise ValueError("align must be positive")
    if x.size and int(x.min()) < 0:
        raise ValueError("aligned slabs need non-negative coordinates")
    coarse = x // align
    cuts = slab_cuts(coarse, world, radius)
    return [c * align for c in cuts]


def coarse_bounds(cmax: Sequence[int], stride: int) -> List[int]:
    """coords_max of the level below a down-sampling layer with kernel size == stride and no padding:
    the last output whose ``stride`` inputs all lie within ``cmax`` (the map builder's bound rule)."""
    return [(int(m) - (stride - 1)) // stride for m in cmax]


def coarsen(coords: torch.Tensor, stride: int, cmax: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Output coordinates of a down-sampling layer with kernel size == stride and no padding: the
    distinct floor(coords / stride), int32 [M,4] sorted by (b, x, y, z), the order in which the map
    builder returns them.  ``cmax`` (the input level's coords_max) drops the outputs beyond
    :func:`coarse_bounds`, as the map builder does."""
    if coords.numel() == 0:
        return coords.clone()
    c = coords.to(torch.int64).clone()
    if int(c[:, 1:].min()) < 0:
        raise ValueError("coarsen needs non-negative coordinates")
    c[:, 1:] = torch.div(c[:, 1:], stride, rounding_mode="floor")
    if cmax is not None:
        bound = torch.tensor(coarse_bounds(cmax, stride), dtype=torch.int64, device=c.device)
        c = c[(c[:, 1:] <= bound).all(dim=1)]
        if c.numel() == 0:
            return c.to(coords.dtype)
    ext = (c.max(dim=0).values + 1).tolist()
    key = ((c[:, 0] * ext[1] + c[:, 1]) * ext[2] + c[:, 2]) * ext[3] + c[:, 3]
    key = torch.unique(key)  # sorted
    out = torch.empty((key.numel(), 4), dtype=torch.int64, device=coords.device)
    out[:, 3] = key % ext[3]
    key = torch.div(key, ext[3], rounding_mode="floor")
    out[:, 2] = key % ext[2]
    key = torch.div(key, ext[2], rounding_mode="floor")
    out[:, 1] = key % ext[1]
    out[:, 0] = torch.div(key, ext[1], rounding_mode="floor")
    return out.to(coords.dtype).contiguous()


class SlabScene:
    """One rank's view of an x-slab decomposition: owned rows first, then the left and right halo.

    ``coords`` / ``feats`` passed in are the rows this rank OWNS (cuts[rank] <= x < cuts[rank+1]).
    ``setup`` exchanges halo coordinates with the two neighbours; ``local_feats`` returns the
    [owned | left halo | right halo] feature matrix after exchanging the boundary rows of ``feats``.
    A submanifold layer run on (local coords, local feats) gives, in its first ``n_owned`` rows,
    exactly the rows a single-GPU run produces for these voxels (same neighbours, same kp order).
    """

    def __init__(self, coords: torch.Tensor, cuts: Sequence[int], rank: int, world: int, radius: int):
        self.rank, self.world, self.radius = rank, world, radius
        self.cuts = list(cuts)
        self.coords = coords
        self.n_owned = int(coords.size(0))
        x = coords[:, 1]
        lo, hi = self.cuts[rank], self.cuts[rank + 1]
        if self.n_owned and (int(x.min()) < lo or int(x.max()) >= hi):
            raise ValueError("coords contain rows outside this rank's slab")
        # rows a neighbour needs from us (our boundary layers)
        self.send_left = torch.nonzero(x < lo + radius).flatten() if rank > 0 else coords.new_zeros((0,), dtype=torch.long)
        self.send_right = torch.nonzero(x >= hi - radius).flatten() if rank < world - 1 else coords.new_zeros((0,), dtype=torch.long)
        self.halo_left = None
        self.halo_right = None
        self.local_coords = None

    # -- point-to-point plumbing (neighbour-only) ---------------------------------------------
    def _exchange(self, to_left, to_right, row_shape, dtype, recv_counts=None, out_left=None, out_right=None):
        """Send a row block to each neighbour, receive theirs; returns (from_left, from_right).
        Without ``recv_counts`` the sizes are exchanged first (one host synchronisation)."""
        dev = self.coords.device
        left, right = self.rank - 1, self.rank + 1
        if recv_counts is None:
            n_send = torch.tensor([0 if to_left is None else to_left.size(0), 0 if to_right is None else to_right.size(0)],
                                  dtype=torch.int64, device=dev)
            n_recv = torch.zeros(2, dtype=torch.int64, device=dev)
            ops = []
            if left >= 0:
                ops += [dist.P2POp(dist.isend, n_send[0:1], left), dist.P2POp(dist.irecv, n_recv[0:1], left)]
            if right < self.world:
                ops += [dist.P2POp(dist.isend, n_send[1:2], right), dist.P2POp(dist.irecv, n_recv[1:2], right)]
            if ops:
                for r in dist.batch_isend_irecv(ops):
                    r.wait()
            recv_counts = n_recv.cpu().tolist()
        from_left = out_left if out_left is not None else torch.empty((recv_counts[0],) + tuple(row_shape), dtype=dtype, device=dev)
        from_right = out_right if out_right is not None else torch.empty((recv_counts[1],) + tuple(row_shape), dtype=dtype, device=dev)
        ops = []
        if left >= 0:
            if to_left.size(0):
                ops.append(dist.P2POp(dist.isend, to_left.contiguous(), left))
            if recv_counts[0]:
                ops.append(dist.P2POp(dist.irecv, from_left, left))
        if right < self.world:
            if to_right.size(0):
                ops.append(dist.P2POp(dist.isend, to_right.contiguous(), right))
            if recv_counts[1]:
                ops.append(dist.P2POp(dist.irecv, from_right, right))
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        return from_left, from_right

    def setup(self):
        """Exchange the halo coordinates (once per scene); the halo sizes are known from then on."""
        if self.world == 1:
            self.halo_left = self.coords[:0]
            self.halo_right = self.coords[:0]
        else:
            self.halo_left, self.halo_right = self._exchange(self.coords[self.send_left], self.coords[self.send_right],
                                                             (4,), self.coords.dtype)
        self.local_coords = torch.cat([self.coords, self.halo_left, self.halo_right], dim=0).contiguous()
        self.n_local = int(self.local_coords.size(0))
        return self

    def alloc_local(self, channels: int, dtype) -> torch.Tensor:
        """An [n_local, channels] feature buffer laid out [owned | left halo | right halo].  A layer
        that writes its output rows into ``buf[:n_owned]`` needs no copy before the next exchange."""
        return torch.empty((self.n_local, channels), dtype=dtype, device=self.coords.device)

    def exchange_into(self, buf: torch.Tensor) -> torch.Tensor:
        """Fill the halo rows of ``buf`` (from :meth:`alloc_local`) with the neighbours' boundary rows
        of their owned part; no size exchange, no host synchronisation, no concatenation."""
        if self.world == 1:
            return buf
        n0, nl = self.n_owned, int(self.halo_left.size(0))
        owned = buf[:n0]
        self._exchange(owned[self.send_left], owned[self.send_right], (buf.size(1),), buf.dtype,
                       recv_counts=[nl, int(self.halo_right.size(0))], out_left=buf[n0:n0 + nl], out_right=buf[n0 + nl:])
        return buf

    def local_feats(self, feats: torch.Tensor) -> torch.Tensor:
        """[owned | left halo | right halo] features from this rank's owned ``feats`` (allocates)."""
        if self.world == 1:
            return feats
        buf = self.alloc_local(feats.size(1), feats.dtype)
        buf[: self.n_owned] = feats
        return self.exchange_into(buf)


class PeerPush:
    """Halo exchange of a :class:`SlabScene` done by the convolution itself.

    Every rank keeps two feature buffers [n_local, C] in symmetric memory (each rank's buffers are
    mapped into its neighbours' address spaces).  A layer reads buffer ``src`` and writes its owned
    output rows into its own buffer ``dst`` AND, from the convolution kernel's epilogue with plain
    peer stores over NVLink, the boundary rows into the halo rows of the neighbours' ``dst`` buffers
    (:meth:`epilogue`).  One barrier between the GPUs (:meth:`barrier`) then makes every ``dst``
    complete; with the two buffers used alternately that barrier also orders the next layer's
    writes after this layer's reads.  Compared with sending the boundary rows after the layer
    (``SlabScene.exchange_into``) there is no gather of the boundary rows, no message and no copy
    into the halo: the rows cross the link while the interior tiles are still being computed.

    The kernels only ever LOAD local memory; remote memory is written, never read, and no multicast
    is involved."""

    def __init__(self, scene: "SlabScene", channels: int, dtype=torch.float16, group=None):
        import torch.distributed._symmetric_memory as symm
        if scene.local_coords is None:
            raise RuntimeError("SlabScene.setup() must run first")
        self.scene, self.channels = scene, channels
        dev = scene.coords.device
        group = group if group is not None else dist.group.WORLD
        nl, nr = int(scene.halo_left.size(0)), int(scene.halo_right.size(0))
        mine = torch.tensor([scene.n_owned, nl, nr, scene.n_local], dtype=torch.int64, device=dev)
        every = [torch.zeros_like(mine) for _ in range(scene.world)]
        dist.all_gather(every, mine, group=group)
        every = [t.cpu().tolist() for t in every]
        rows = max(e[3] for e in every)
        self.buffers = [symm.empty((rows, channels), dtype=dtype, device=dev) for _ in range(2)]
        self.handles = [symm.rendezvous(t, group) for t in self.buffers]
        # where my boundary rows live in the neighbours' buffers
        n0 = scene.n_owned
        self.slots = [torch.full((n0,), -1, dtype=torch.int32, device=dev) for _ in range(2)]
        if scene.rank > 0:  # my left boundary = the left neighbour's RIGHT halo
            e = every[scene.rank - 1]
            self.slots[0][scene.send_left] = (e[0] + e[1] + torch.arange(scene.send_left.numel(), device=dev)).to(torch.int32)
        if scene.rank < scene.world - 1:  # my right boundary = the right neighbour's LEFT halo
            e = every[scene.rank + 1]
            self.slots[1][scene.send_right] = (e[0] + torch.arange(scene.send_right.numel(), device=dev)).to(torch.int32)

    def local(self, k: int) -> torch.Tensor:
        """Buffer ``k`` as this rank's [n_local, C] feature matrix ([owned | left halo | right halo])."""
        return self.buffers[k][: self.scene.n_local]

    def owned(self, k: int) -> torch.Tensor:
        return self.buffers[k][: self.scene.n_owned]

    def epilogue(self, k: int, **kwargs):
        """A FusedEpilogue (plus any of its usual fields) that also stores the boundary rows into the
        neighbours' buffer ``k``."""
        from .functional import FusedEpilogue
        r, w = self.scene.rank, self.scene.world
        ptrs = self.handles[k].buffer_ptrs
        bases = (int(ptrs[r - 1]) if r > 0 else 0, int(ptrs[r + 1]) if r < w - 1 else 0)
        return FusedEpilogue(push_slots=(self.slots[0] if bases[0] else None, self.slots[1] if bases[1] else None),
                             push_bases=bases, **kwargs)

    def barrier(self, k: int) -> None:
        """All ranks have finished the layer that wrote buffer ``k`` (queued on the current stream)."""
        self.handles[k].barrier(channel=0)


class SlabLevels:
    """A slab decomposition of every coordinate level of a network with down-/up-sampling layers.

    ``coords`` are the rows this rank owns at the finest level, ``cuts`` come from
    :func:`aligned_slab_cuts` with ``align`` = the product of ``strides``, ``cmax`` is the whole scene's
    coords_max (``cmax[l]`` afterwards: the same per level).  ``scenes[l]`` is the
    :class:`SlabScene` of level l (level l+1 = level l down-sampled by ``strides[l]`` with kernel size ==
    stride and no padding): its owned rows are exactly the level's voxels inside this rank's slab, in the
    order a map builder returns them, and its halo (exchanged once, here) serves the level's submanifold
    layers.  Because every cut is a multiple of the level's stride, all children of a coarse voxel belong
    to the rank that owns it: the down-sampling layer and its transposed layer run on
    (``scenes[l].coords`` -> ``scenes[l+1].coords``) with no exchange at all, and what they return for the
    owned rows is what an undivided run returns for those voxels."""

    def __init__(self, coords: torch.Tensor, cuts: Sequence[int], rank: int, world: int, radius: int,
                 strides: Sequence[int], cmax: Sequence[int]):
        self.strides = [int(s) for s in strides]
        self.scenes: List[SlabScene] = []
        self.cmax: List[List[int]] = []  # the WHOLE scene's coords_max per level (what every map is built with)
        level_cuts, level_cmax = [int(c) for c in cuts], [int(m) for m in cmax]
        for l in range(len(self.strides) + 1):
            self.scenes.append(SlabScene(coords, level_cuts, rank, world, radius).setup())
            self.cmax.append(level_cmax)
            if l < len(self.strides):
                s = self.strides[l]
                if s < 1 or any(c % s for c in level_cuts):
                    raise ValueError("slab cuts must be multiples of the cumulative stride (aligned_slab_cuts)")
                coords = coarsen(coords, s, level_cmax)
                level_cuts = [c // s for c in level_cuts]
                level_cmax = coarse_bounds(level_cmax, s)

    def __len__(self) -> int:
        return len(self.scenes)

    def __getitem__(self, level: int) -> SlabScene:
        return self.scenes[level]

    # Halo rows travel through symmetric-memory mailboxes (HaloMailbox) where that is available, else as
    # messages (SlabScene.exchange_into); set to False to use messages throughout.
    use_mailboxes = True

    def exchange_into(self, level: int, buf: torch.Tensor) -> torch.Tensor:
        """Fill the halo rows of ``buf`` ([owned | halo] rows of ``level``) from the neighbouring ranks."""
        scene = self.scenes[level]
        if scene.world == 1:
            return buf
        row_bytes = buf.size(1) * buf.element_size()
        if self.use_mailboxes and buf.is_cuda and row_bytes % 16 == 0 and (buf.stride(0) * buf.element_size()) % 16 == 0:
            boxes = self.__dict__.setdefault("_mailboxes", {})
            key = (level, buf.size(1), buf.dtype)
            if key not in boxes:
                try:   # (collective: every rank reaches this for the same layer)
                    boxes[key] = HaloMailbox(scene, buf.size(1), buf.dtype)
                except Exception:  # no symmetric memory on this system
                    boxes[key] = None
            if boxes[key] is not None:
                return boxes[key].exchange_into(buf)
        return scene.exchange_into(buf)

    def level_of(self, stride: Sequence[int]) -> int:
        """The level whose voxels are ``stride`` finest-level voxels wide (the same along x, y, z)."""
        s = [int(v) for v in stride]
        total = 1
        for level in range(len(self.scenes)):
            if s == [total] * 3:
                return level
            if level < len(self.strides):
                total *= self.strides[level]
        raise ValueError(f"no slab level with stride {s}")


class HaloMailbox:
    """Halo exchange of a :class:`SlabScene` without messages, for feature matrices of one width and dtype.

    Every rank keeps two mailboxes [halo rows, C] in symmetric memory, laid out like the halo part of a local
    feature matrix ([from the left | from the right]).  ``exchange_into(buf)`` stores this rank's boundary rows
    straight into the neighbours' mailboxes (``pce_push_rows``: plain peer stores over NVLink, nothing is loaded
    from a peer and no multicast is involved), passes one barrier between the GPUs, and copies its own mailbox
    behind the owned rows of ``buf``.  The two mailboxes alternate, so the barrier of one exchange also orders
    the next exchange's stores after this exchange's copy."""

    def __init__(self, scene: "SlabScene", channels: int, dtype=torch.float16, group=None):
        import torch.distributed._symmetric_memory as symm
        if scene.local_coords is None:
            raise RuntimeError("SlabScene.setup() must run first")
        if (channels * torch.empty((), dtype=dtype).element_size()) % 16:
            raise ValueError("a mailbox row must be a multiple of 16 bytes")
        self.scene, self.channels, self.dtype = scene, channels, dtype
        dev = scene.coords.device
        group = group if group is not None else dist.group.WORLD
        self.nl, self.nr = int(scene.halo_left.size(0)), int(scene.halo_right.size(0))
        mine = torch.tensor([self.nl, self.nr], dtype=torch.int64, device=dev)
        every = [torch.zeros_like(mine) for _ in range(scene.world)]
        dist.all_gather(every, mine, group=group)
        self.every = [t.cpu().tolist() for t in every]
        rows = max(max(e[0] + e[1] for e in self.every), 1)
        self.boxes = [symm.empty((rows, channels), dtype=dtype, device=dev) for _ in range(2)]
        self.handles = [symm.rendezvous(t, group) for t in self.boxes]
        self.send_left = scene.send_left.to(torch.int32).contiguous()
        self.send_right = scene.send_right.to(torch.int32).contiguous()
        self.k = 0

    def exchange_into(self, buf: torch.Tensor) -> torch.Tensor:
        from . import _lib
        sc = self.scene
        if buf.size(1) != self.channels or buf.dtype != self.dtype or buf.size(0) != sc.n_local or buf.stride(1) != 1:
            raise ValueError("the buffer is not an [n_local, C] matrix of this mailbox's width and type")
        k, self.k = self.k, self.k ^ 1
        row_bytes = self.channels * buf.element_size()
        pitch = buf.stride(0) * buf.element_size()
        stream = _lib.stream_ptr(buf.device)
        ptrs = self.handles[k].buffer_ptrs
        if sc.rank > 0 and self.send_left.numel():    # my left boundary: the left neighbour's rows "from the right"
            dst = int(ptrs[sc.rank - 1]) + self.every[sc.rank - 1][0] * row_bytes
            _lib.check(_lib.lib.pce_push_rows(buf.data_ptr(), pitch, self.send_left.data_ptr(), self.send_left.numel(),
                                              row_bytes, dst, row_bytes, stream), "pce_push_rows")
        if sc.rank < sc.world - 1 and self.send_right.numel():  # my right boundary: the right neighbour's rows "from the left"
            _lib.check(_lib.lib.pce_push_rows(buf.data_ptr(), pitch, self.send_right.data_ptr(), self.send_right.numel(),
                                              row_bytes, int(ptrs[sc.rank + 1]), row_bytes, stream), "pce_push_rows")
        self.handles[k].barrier(channel=0)
        n = self.nl + self.nr
        if n:
            buf[sc.n_owned: sc.n_owned + n].copy_(self.boxes[k][:n])
        return buf


def split_scene(coords: np.ndarray, world: int, radius: int, align: int = 1):
    """Host-side split of a whole scene (int32 [N,4]) into per-rank owned row indices + the cuts
    (multiples of ``align``: see :func:`aligned_slab_cuts`)."""
    cuts = aligned_slab_cuts(coords[:, 1], world, radius, align) if align > 1 else slab_cuts(coords[:, 1], world, radius)
    owned = [np.nonzero((coords[:, 1] >= cuts[g]) & (coords[:, 1] < cuts[g + 1]))[0] for g in range(world)]
    return cuts, owned
