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
