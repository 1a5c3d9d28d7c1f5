"""Multi-rank host logic on CPU with the gloo backend (world_size 2 and 3): scan sharding, the
max-over-ranks reduction and the slab decomposition with its neighbour-only halo exchange.  The
convolution itself is done by the CPU oracle here, which checks the decomposition exactly: the owned
rows of every slab equal the rows of the undivided scene."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import conv_oracle as co
from oracle import kmap_oracle as ko
from tests.helpers import cmax_of, surface_cloud


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ks, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pcengine_b200 import multigpu as mg
        # --- scan sharding + reduction ---
        mine = mg.scans_for_rank(8, rank, world)
        assert mg.max_over_ranks(float(rank + 1)) == float(world)
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        assert sorted(sum(gathered, [])) == list(range(8))
        # --- slab decomposition of one scene ---
        coords = surface_cloud(77, 48, batch=1)
        torch.manual_seed(5)
        feats = torch.randn(len(coords), 8)
        w = torch.randn(ks ** 3, 8, 6) / 10
        radius = (ks - 1) // 2
        cuts, owned = mg.split_scene(coords, world, radius)
        idx = owned[rank]
        scene = mg.SlabScene(torch.from_numpy(coords[idx]), cuts, rank, world, radius).setup()
        local = scene.local_feats(feats[idx])
        lc = scene.local_coords.numpy()
        assert len(np.unique(lc, axis=0)) == len(lc)          # halo rows are not owned rows
        d2 = ko.build_d2(lc, (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
        out_local = co.conv_forward(local, w, d2)[: scene.n_owned]
        # reference: the undivided scene
        d2f = ko.build_d2(coords, (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
        full = co.conv_forward(feats, w, d2f)
        assert torch.allclose(out_local, full[idx], rtol=0, atol=1e-5)
        # halo sizes are a small fraction and symmetric between neighbours
        sizes = [None] * world
        dist.all_gather_object(sizes, (len(scene.send_left), len(scene.send_right), len(scene.halo_left), len(scene.halo_right)))
        for g in range(world - 1):
            assert sizes[g][1] == sizes[g + 1][2] and sizes[g + 1][0] == sizes[g][3]
        out_q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        out_q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def _levels_worker(rank, world, port, out_q):
    """A small U-shaped network (3x3x3 -> 2x2x2 stride 2 -> 3x3x3 -> transposed 2x2x2 -> 3x3x3) on slabs whose
    cuts are multiples of the stride: only the submanifold layers exchange rows."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pcengine_b200 import multigpu as mg
        coords = surface_cloud(78, 63, batch=1)   # odd extent: the bound rule drops the last coarse plane
        cm = cmax_of(coords)
        torch.manual_seed(6)
        feats = torch.randn(len(coords), 8)
        w0, wd, w1, wu, w2 = (torch.randn(27, 8, 8) / 10, torch.randn(8, 8, 12) / 4, torch.randn(27, 12, 12) / 10,
                              torch.randn(8, 12, 8) / 4, torch.randn(27, 8, 6) / 10)
        sub, down = ((3, 3, 3), (1, 1, 1)), ((2, 2, 2), (2, 2, 2))
        z = (0, 0, 0)
        # the undivided scene
        d0 = ko.build_d2(coords, *sub, z, [0, 0, 0], cm, True)
        dd = ko.build_d2(coords, *down, z, [0, 0, 0], cm, False)
        d1 = ko.build_d2(dd["out_coords"], *sub, z, [0, 0, 0], dd["cmax_out"], True)
        a = co.conv_forward(feats, w0, d0)
        b = co.conv_forward(a, wd, dd)
        c = co.conv_forward(b, w1, d1)
        u = co.conv_forward(c, wu, dd, transposed=True)
        y = co.conv_forward(u, w2, d0)
        # slabs
        cuts, owned = mg.split_scene(coords, world, 1, align=2)
        assert all(k % 2 == 0 for k in cuts)
        idx = owned[rank]
        levels = mg.SlabLevels(torch.from_numpy(coords[idx]), cuts, rank, world, 1, [2], cm)
        s0, s1 = levels[0], levels[1]
        assert len(levels) == 2 and levels.cmax == [list(cm), list(dd["cmax_out"])]
        l0 = ko.build_d2(s0.local_coords.numpy(), *sub, z, [0, 0, 0], cm, True)
        ld = ko.build_d2(coords[idx], *down, z, [0, 0, 0], cm, False)          # owned rows only: no halo
        assert np.array_equal(ld["out_coords"], s1.coords.numpy())
        l1 = ko.build_d2(s1.local_coords.numpy(), *sub, z, [0, 0, 0], levels.cmax[1], True)
        a_l = co.conv_forward(s0.local_feats(feats[idx]), w0, l0)[: s0.n_owned]
        b_l = co.conv_forward(a_l, wd, ld)
        c_l = co.conv_forward(s1.local_feats(b_l), w1, l1)[: s1.n_owned]
        u_l = co.conv_forward(c_l, wu, ld, transposed=True)
        y_l = co.conv_forward(s0.local_feats(u_l), w2, l0)[: s0.n_owned]
        lut = {tuple(r): i for i, r in enumerate(dd["out_coords"].tolist())}
        idx1 = [lut[tuple(r)] for r in s1.coords.tolist()]
        assert torch.allclose(b_l, b[idx1], rtol=0, atol=1e-5) and torch.allclose(c_l, c[idx1], rtol=0, atol=1e-5)
        assert torch.allclose(u_l, u[idx], rtol=0, atol=1e-5) and torch.allclose(y_l, y[idx], rtol=0, atol=1e-5)
        # every coarse voxel is owned by exactly one rank
        counts = [None] * world
        dist.all_gather_object(counts, s1.n_owned)
        assert sum(counts) == len(dd["out_coords"])
        out_q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        out_q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_down_and_up_sampling_layers_on_aligned_slabs(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_levels_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def _deep_worker(rank, world, port, out_q):
    """Three coordinate levels (strides 2, 2; cuts at multiples of 4): down, down, 3x3x3 at the coarsest level,
    up, up, 3x3x3 at the finest, every strided layer on owned rows only."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pcengine_b200 import multigpu as mg
        coords = surface_cloud(80, 62, batch=1)
        cm = cmax_of(coords)
        torch.manual_seed(7)
        feats = torch.randn(len(coords), 6)
        wd0, wd1, w2, wu1, wu0, w0 = (torch.randn(8, 6, 8) / 4, torch.randn(8, 8, 10) / 4, torch.randn(27, 10, 10) / 10,
                                      torch.randn(8, 10, 8) / 4, torch.randn(8, 8, 6) / 4, torch.randn(27, 6, 5) / 10)
        sub, down, z = ((3, 3, 3), (1, 1, 1)), ((2, 2, 2), (2, 2, 2)), (0, 0, 0)

        def run(c0, f, local0=None, local2=None, grow0=lambda t: t, grow2=lambda t: t, n0=None, n2=None):
            m01 = ko.build_d2(c0, *down, z, [0, 0, 0], cm, False)
            m12 = ko.build_d2(m01["out_coords"], *down, z, [0, 0, 0], m01["cmax_out"], False)
            s2 = ko.build_d2(m12["out_coords"] if local2 is None else local2, *sub, z, [0, 0, 0], m12["cmax_out"], True)
            s0 = ko.build_d2(c0 if local0 is None else local0, *sub, z, [0, 0, 0], cm, True)
            a = co.conv_forward(f, wd0, m01)
            b = co.conv_forward(a, wd1, m12)
            c = co.conv_forward(grow2(b), w2, s2)[: (n2 if n2 is not None else len(b))]
            d = co.conv_forward(c, wu1, m12, transposed=True)
            e = co.conv_forward(d, wu0, m01, transposed=True)
            y = co.conv_forward(grow0(e), w0, s0)[: (n0 if n0 is not None else len(e))]
            return m12["out_coords"], c, y
        coarse, c_full, y_full = run(coords, feats)
        cuts, owned = mg.split_scene(coords, world, 1, align=4)
        idx = owned[rank]
        levels = mg.SlabLevels(torch.from_numpy(coords[idx]), cuts, rank, world, 1, [2, 2], cm)
        assert len(levels) == 3 and all(k % 4 == 0 for k in cuts)
        mine, c_l, y_l = run(coords[idx], feats[idx], levels[0].local_coords.numpy(), levels[2].local_coords.numpy(),
                             levels[0].local_feats, levels[2].local_feats, levels[0].n_owned, levels[2].n_owned)
        assert np.array_equal(mine, levels[2].coords.numpy())
        lut = {tuple(r): i for i, r in enumerate(coarse.tolist())}
        idx2 = [lut[tuple(r)] for r in mine.tolist()]
        assert torch.allclose(c_l, c_full[idx2], rtol=0, atol=1e-5) and torch.allclose(y_l, y_full[idx], rtol=0, atol=1e-5)
        out_q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        out_q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_three_levels_on_aligned_slabs():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_deep_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def test_aligned_cuts_and_coarsening():
    from pcengine_b200 import multigpu as mg
    rng = np.random.default_rng(1)
    x = rng.integers(0, 1000, 50000)
    cuts = mg.aligned_slab_cuts(x, 4, 1, 8)
    assert len(cuts) == 5 and all(c % 8 == 0 for c in cuts) and cuts[0] <= x.min() and cuts[-1] > x.max()
    assert all(b - a >= 8 for a, b in zip(cuts[:-1], cuts[1:]))
    with pytest.raises(ValueError):
        mg.aligned_slab_cuts(np.array([-1, 5]), 2, 1, 2)
    coords = surface_cloud(79, 47, batch=2)
    cm = cmax_of(coords)
    d = ko.build_d2(coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], cm, False)
    assert np.array_equal(mg.coarsen(torch.from_numpy(coords), 2, cm).numpy(), d["out_coords"])
    assert mg.coarse_bounds(cm, 2) == list(d["cmax_out"])
    assert (cm[0] + 1) % 2 == 1
    one = mg.SlabLevels(torch.from_numpy(coords), [0, cm[0] + 2], 0, 1, 1, [2], cm)   # one slab: nothing to exchange
    assert np.array_equal(one[1].coords.numpy(), d["out_coords"]) and one[1].n_local == one[1].n_owned
    with pytest.raises(ValueError, match="multiples"):
        mg.SlabLevels(torch.from_numpy(coords), [0, cm[0] + 1], 0, 1, 1, [2], cm)      # an odd cut under stride 2


@pytest.mark.parametrize("world,ks", [(2, 3), (3, 5)])
def test_slabs_and_sharding_under_gloo(world, ks):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ks, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def test_slab_cuts_balance_and_width():
    from pcengine_b200 import multigpu as mg
    rng = np.random.default_rng(0)
    x = rng.integers(0, 2000, 100000)
    cuts = mg.slab_cuts(x, 8, 2)
    counts = np.histogram(x, bins=cuts)[0]
    assert len(cuts) == 9 and counts.sum() == len(x) and counts.max() / counts.mean() < 1.05
    with pytest.raises(ValueError):
        mg.slab_cuts(np.array([0, 1, 2]), 4, 2)
    assert mg.scans_for_rank(8, 2, 3) == [6, 7] and mg.scans_for_rank(8, 0, 3) == [0, 1, 2]
