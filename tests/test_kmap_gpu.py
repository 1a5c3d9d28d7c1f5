"""Kernel maps from the CUDA path must equal the oracle's bit for bit (GPU)."""
import numpy as np
import pytest
import torch

from oracle import kmap_oracle as ko
from tests.helpers import cmax_of, random_cloud, surface_cloud

pytestmark = pytest.mark.gpu


def _check(coords, ks, stride, pad, subm):
    import pcengine_b200 as pce
    dev = torch.device("cuda:0")
    cmax_in = cmax_of(coords)
    d2 = ko.build_d2(coords, ks, stride, pad, [0, 0, 0], cmax_in, subm)
    km = pce.KernelMap(torch.from_numpy(coords).to(dev), ks, stride, pad, [0, 0, 0], d2["cmax_out"], subm)
    assert km.n_out == d2["n_out"]
    assert np.array_equal(km.out_coords.cpu().numpy().reshape(-1, 4), d2["out_coords"].reshape(-1, 4))
    assert np.array_equal(km.map.cpu().numpy(), d2["map"])
    assert np.array_equal(km.knnz.cpu().numpy(), d2["knnz"])
    assert np.array_equal(km.kpos.cpu().numpy(), d2["kpos"])
    assert np.array_equal(km.qkpos.cpu().numpy(), d2["qkpos"])
    p, q = km.sizes()
    assert p == len(d2["imap"]) and q == d2["qsum"]
    imap, omap = km.pairs()
    assert np.array_equal(imap.cpu().numpy(), d2["imap"])
    assert np.array_equal(omap.cpu().numpy(), d2["omap"])
    d1 = ko.build_d1(d2)
    imap_c, icsr, omap_c, ocsr = km.d1()
    assert np.array_equal(icsr.cpu().numpy(), d1["icsr"])
    assert np.array_equal(ocsr.cpu().numpy(), d1["ocsr"])
    assert np.array_equal(imap_c.cpu().numpy(), d1["imap"])
    assert np.array_equal(omap_c.cpu().numpy(), d1["omap"])
    for tr in (False, True):
        nb = ko.neighbour_csr(d2, transposed=tr)
        csr = km.csr(transposed=tr)
        total = int(nb["rowptr"][-1])
        assert np.array_equal(csr.rowptr.cpu().numpy(), nb["rowptr"])
        assert np.array_equal(csr.mask.cpu().numpy().view(np.uint32)[: nb["n_out"]], nb["mask"])
        assert np.array_equal(csr.nbr.cpu().numpy()[:total], nb["nbr"])
    # the pair-list route used by the drop-in conv entry point gives the same CSR
    from pcengine_b200.kmap import csr_from_pairs
    nb = ko.neighbour_csr(d2)
    c2 = csr_from_pairs(omap, imap, km.kpos, km.kv, km.n_out, km.n_in, km.mid if subm else -1)
    assert np.array_equal(c2.rowptr.cpu().numpy(), nb["rowptr"])
    assert np.array_equal(c2.mask.cpu().numpy().view(np.uint32)[: nb["n_out"]], nb["mask"])
    assert np.array_equal(c2.nbr.cpu().numpy()[: int(nb["rowptr"][-1])], nb["nbr"])
    return d2


@pytest.mark.parametrize("ks", [(3, 3, 3), (5, 5, 5), (2, 2, 2), (3, 1, 5), (1, 1, 1)])
def test_submanifold_random(ks):
    _check(random_cloud(1, 24, 3000, batch=2), ks, (1, 1, 1), (0, 0, 0), True)


def test_submanifold_config1_shape():
    """20,000 voxels in 64^3 (the fp32 C=16 benchmark case)."""
    from pcengine_b200 import synth
    coords = synth.with_batch(synth.uniform_grid(20000, 64, 1001))
    d2 = _check(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), True)
    assert d2["n_in"] == 20000


def test_submanifold_surface():
    _check(surface_cloud(4, 96, batch=2), (3, 3, 3), (1, 1, 1), (0, 0, 0), True)


@pytest.mark.parametrize("ks,stride,pad", [((2, 2, 2), (2, 2, 2), (0, 0, 0)), ((3, 3, 3), (2, 2, 2), (0, 0, 0)),
                                           ((3, 3, 3), (2, 2, 2), (1, 1, 1)), ((2, 2, 2), (1, 2, 2), (0, 0, 0)),
                                           ((3, 3, 3), (3, 3, 3), (0, 0, 0)), ((2, 3, 2), (2, 1, 2), (0, 1, 0)),
                                           ((5, 5, 5), (2, 2, 2), (2, 2, 2)), ((4, 4, 4), (2, 2, 2), (1, 1, 1)),
                                           ((5, 5, 5), (3, 3, 3), (0, 0, 0)), ((4, 2, 5), (3, 2, 2), (1, 0, 2))])
def test_strided(ks, stride, pad):
    _check(random_cloud(2, 30, 4000, batch=2), ks, stride, pad, False)
    _check(surface_cloud(5, 64), ks, stride, pad, False)


def test_degenerate_inputs():
    one = np.array([[0, 5, 5, 5]], np.int32)
    _check(one, (3, 3, 3), (1, 1, 1), (0, 0, 0), True)
    _check(one, (2, 2, 2), (2, 2, 2), (0, 0, 0), False)
    # isolated voxels: no neighbour anywhere
    iso = np.array([[0, 4 * i, 4 * j, 4 * k] for i in range(5) for j in range(5) for k in range(5)], np.int32)
    d2 = _check(iso, (3, 3, 3), (1, 1, 1), (0, 0, 0), True)
    assert d2["kpos"][-1] == 0
    # fully dense block: every interior voxel has all 27
    blk = np.array([[0, i, j, k] for i in range(9) for j in range(9) for k in range(9)], np.int32)
    d2 = _check(blk, (3, 3, 3), (1, 1, 1), (0, 0, 0), True)
    assert d2["knnz"][0] == 8 ** 3
    # coordinates at zero and far out, several batches
    far = np.array([[0, 0, 0, 0], [0, 0, 0, 1], [1, 3000, 3000, 100], [1, 3000, 3001, 100], [2, 0, 0, 0]], np.int32)
    _check(far, (3, 3, 3), (1, 1, 1), (0, 0, 0), True)
    _check(far, (2, 2, 2), (2, 2, 2), (0, 0, 0), False)


def test_out_of_range_coordinate_reports_status():
    import pcengine_b200 as pce
    bad = torch.tensor([[0, 1, 1, 1], [0, 70000, 1, 1]], dtype=torch.int32, device="cuda:0")
    km = pce.KernelMap(bad, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], [70000, 1, 1], True)
    with pytest.raises(RuntimeError):
        km.sizes()


@pytest.mark.parametrize("ks,sort_rows,tile_rows,identity,slots", [
    ((3, 3, 3), True, 128, False, 1), ((3, 3, 3), False, 128, False, 1), ((5, 5, 5), True, 128, False, 1),
    ((2, 2, 2), True, 128, False, 1), ((3, 3, 3), True, 256, False, 1), ((5, 5, 5), False, 256, False, 1),
    ((3, 3, 3), True, 128, True, 1), ((3, 3, 3), True, 256, True, 1), ((3, 3, 3), True, 128, False, 2),
    ((3, 3, 3), True, 128, True, 4), ((5, 5, 5), True, 256, True, 2), ((2, 2, 2), False, 128, False, 4),
    ((3, 3, 3), True, 512, False, 1), ((5, 5, 5), True, 512, True, 1)])
def test_tile_lists_match_the_csr(ks, sort_rows, tile_rows, identity, slots):
    """Tile lists are the oracle's neighbour CSR re-laid: per tile of 128, 256 or 512 rows (in processing
    order) one stage per offset present in the tile, with each row's neighbour at that offset or -1;
    with ``identity`` one more stage (offset -1) in which every row names itself; with ``slots`` > 1 the
    tile's offsets are taken ``slots`` per stage (unused slots: offset -2, rows -1); with one offset per
    stage the entry also says, in bit 8+s, whether the tile's s-th 128-row sub-tile has the offset."""
    import pcengine_b200 as pce
    coords = surface_cloud(14, 56, batch=2)
    d2 = ko.build_d2(coords, ks, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    nb = ko.neighbour_csr(d2)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), ks, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    csr = km.csr()
    csr.tiles(sort_rows, tile_rows, identity, slots)
    _, order, tile_ptr, stage_kp, stage_nbr = csr._tiles[(sort_rows, tile_rows, identity, slots)][:5]
    order, tile_ptr = order.cpu().numpy(), tile_ptr.cpu().numpy()
    stage_kp, stage_nbr = stage_kp.cpu().numpy(), stage_nbr.cpu().numpy().reshape(-1, tile_rows)
    stage_kp3, stage_nbr3 = stage_kp.reshape(-1, slots), stage_nbr.reshape(-1, slots, tile_rows)
    n, kv = km.n_out, km.kv
    assert np.array_equal(np.sort(order), np.arange(n))
    if not sort_rows:
        assert np.array_equal(order, np.arange(n))
    # dense view of the oracle CSR: want[row, kp] = input row or -1
    want = np.full((n, kv), -1, np.int64)
    rows = np.repeat(np.arange(n), np.diff(nb["rowptr"]))
    kps = np.concatenate([np.nonzero([(int(nb["mask"][r, k // 32]) >> (k % 32)) & 1 for k in range(kv)])[0]
                          for r in range(n)])
    want[rows, kps] = nb["nbr"]
    n_tiles = (n + tile_rows - 1) // tile_rows
    assert tile_ptr[0] == 0 and len(tile_ptr) == n_tiles + 1
    for t in range(n_tiles):
        rws = order[t * tile_rows:(t + 1) * tile_rows]
        present = np.nonzero((want[rws] >= 0).any(axis=0))[0]
        a, b = tile_ptr[t], tile_ptr[t + 1]
        if identity:
            b -= 1
            assert stage_kp3[b, 0] == -1 and (stage_kp3[b, 1:] == -2).all()
            assert np.array_equal(stage_nbr3[b, 0, :len(rws)], rws) and (stage_nbr3[b, 0, len(rws):] == -1).all()
            assert (stage_nbr3[b, 1:] == -1).all()
        assert b - a == (len(present) + slots - 1) // slots
        kps = stage_kp3[a:b].reshape(-1).copy()
        nbrs = stage_nbr3[a:b].reshape(-1, tile_rows)
        if slots == 1:  # offset in the low byte, sub-tile presence above it
            has = want[rws][:, present] >= 0                                   # [rows of the tile, present offsets]
            has = np.concatenate([has, np.zeros((tile_rows - len(rws), len(present)), bool)])
            bits = has.reshape(tile_rows // 128, 128, -1).any(axis=1)            # [sub-tile, offset]
            want_bits = (bits * (1 << np.arange(tile_rows // 128))[:, None]).sum(axis=0)
            assert np.array_equal(kps[:len(present)] >> 8, want_bits)
            kps[:len(present)] &= 255
        assert np.array_equal(kps[:len(present)], present) and (kps[len(present):] == -2).all()
        assert np.array_equal(nbrs[:len(present), :len(rws)], want[rws][:, present].T)
        assert (nbrs[:len(present), len(rws):] == -1).all() and (nbrs[len(present):] == -1).all()


@pytest.mark.parametrize("ks", [(3, 3, 3), (5, 5, 5), (4, 4, 4), (2, 2, 2)])
def test_row_order_groups_equal_masks_and_rare_offsets(ks):
    """The processing order is a permutation in which rows with the same indicator bitmask are
    contiguous, and the rows that have the rarest offset form one contiguous run at the end (that
    offset is the most significant bit of the sort key), for one-, two- and four-word masks."""
    import pcengine_b200 as pce
    coords = surface_cloud(17, 48, batch=2)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), ks, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    csr = km.csr()
    order = csr.order().cpu().numpy()
    n, kv = km.n_out, km.kv
    assert np.array_equal(np.sort(order), np.arange(n))
    mask = csr.mask.cpu().numpy().view(np.uint32)
    bits = np.zeros((n, kv), dtype=bool)
    for k in range(kv):
        bits[:, k] = (mask[:, k // 32] >> (k % 32)) & 1
    sorted_bits = bits[order]
    changes = np.count_nonzero((sorted_bits[1:] != sorted_bits[:-1]).any(axis=1))
    assert changes == len(np.unique(bits, axis=0)) - 1
    counts = bits.sum(0)
    present = np.nonzero(counts)[0]
    rarest = present[np.argmin(counts[present])]  # ties: lowest index, as the kernel ranks them
    has = sorted_bits[:, rarest]
    absent_rank = [k for k in range(kv) if counts[k] < counts[rarest]]  # offsets no row has rank above it
    if not absent_rank or all(counts[k] == 0 for k in absent_rank):
        assert has[-int(counts[rarest]):].all() and not has[:-int(counts[rarest])].any()


@pytest.mark.parametrize("n,voxel", [(50000, 0.05), (20000, (0.1, 0.05, 0.2)), (1, 0.5), (3000, 1)])
def test_device_voxelisation_matches_the_host_path(n, voxel):
    """sparse_quantize on a CUDA tensor returns what the NumPy path returns: the same voxels in the
    same order, the first point of every voxel, and the point-to-voxel map (negative coordinates,
    many points per voxel, anisotropic voxels)."""
    import pcengine_b200 as pce
    rng = np.random.default_rng(n)
    pts = (rng.normal(0, 3.0, (n, 3)) + rng.integers(-2, 3, (n, 3))).astype(np.float32)
    pts[: n // 4] = pts[n // 4: 2 * (n // 4)]  # exact duplicates
    want_c, want_i, want_v = pce.sparse_quantize(pts, voxel, return_index=True, return_inverse=True)
    got_c, got_i, got_v = pce.sparse_quantize(torch.from_numpy(pts).cuda(), voxel, return_index=True, return_inverse=True)
    assert got_c.dtype == torch.int32 and got_c.is_cuda and got_c.is_contiguous()
    assert np.array_equal(got_c.cpu().numpy(), want_c)
    assert np.array_equal(got_i.cpu().numpy(), want_i)
    assert np.array_equal(got_v.cpu().numpy(), want_v)
    only = pce.sparse_quantize(torch.from_numpy(pts).cuda(), voxel)
    assert torch.equal(only, got_c)
    # the voxels feed a kernel map directly
    coords = torch.cat([torch.zeros((got_c.size(0), 1), dtype=torch.int32, device="cuda"), got_c - got_c.min(0).values], dim=1)
    km = pce.KernelMap(coords.contiguous(), (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0],
                       coords[:, 1:].max(0).values.tolist(), True)
    assert km.sizes()[0] >= 0


def test_device_voxelisation_edge_cases():
    import pcengine_b200 as pce
    empty = pce.sparse_quantize(torch.empty((0, 3), device="cuda"), 0.1, return_inverse=True)
    assert empty[0].shape == (0, 3) and empty[1].shape == (0,)
    with pytest.raises(RuntimeError):  # 1e9 / 0.01 does not fit the packable coordinate range
        pce.sparse_quantize(torch.tensor([[1e9, 0.0, 0.0]], device="cuda"), 0.01)
    with pytest.raises(NotImplementedError):
        pce.sparse_quantize(torch.zeros((4, 3), dtype=torch.float64, device="cuda"), 0.1)


def test_cooperative_query_builds_the_same_maps():
    """Four lanes per query (64-byte probe rounds, ballots) and one thread per query give identical
    kernel maps: submanifold (mirrored probes), strided with the transposed table, 5x5x5."""
    import pcengine_b200 as pce
    from pcengine_b200 import _lib
    coords = surface_cloud(19, 80, batch=2)
    cd = torch.from_numpy(coords).cuda()
    cmax = cmax_of(coords)
    cases = [((3, 3, 3), (1, 1, 1), True, cmax), ((5, 5, 5), (1, 1, 1), True, cmax),
             ((2, 2, 2), (2, 2, 2), False, [(c - 1) // 2 for c in cmax]), ((3, 3, 3), (2, 2, 2), False, [(c - 2) // 2 for c in cmax])]
    for ks, stride, subm, cm in cases:
        maps = []
        try:
            for lanes4 in (0, 1):
                _lib.lib.pce_tune(5, lanes4)
                km = pce.KernelMap(cd, ks, stride, (0, 0, 0), [0, 0, 0], cm, subm)
                maps.append((km.map.clone(), None if km.map_out is None else km.map_out.clone(), km.knnz.clone(), km.kpos.clone()))
        finally:
            _lib.lib.pce_tune(5, 0)
        for a, b in zip(*maps):
            assert (a is None and b is None) or torch.equal(a, b)
        d2 = ko.build_d2(coords, ks, stride, (0, 0, 0), [0, 0, 0], cmax, subm)
        assert np.array_equal(maps[1][0].cpu().numpy(), d2["map"].reshape(-1))
