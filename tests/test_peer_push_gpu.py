"""Slab-parallel scene on two GPUs with the halo exchange done by the convolution's epilogue
(peer stores into the neighbours' symmetric-memory buffers): the owned rows of every slab must be
bit-identical to the undivided scene after two chained layers.  Needs two GPUs; skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF, multigpu as mg, synth
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        xyz, _ = synth.indoor_room(3001, 60000)
        coords_h = synth.with_batch(xyz)
        cmax = coords_h[:, 1:].max(0).tolist()
        c, ks, radius = 64, 3, 1
        g = torch.Generator().manual_seed(5)
        feats_all = torch.randn(len(coords_h), c, generator=g).half()
        ws = [(torch.randn(27, c, c, generator=g) / (27 * c) ** 0.5).half().to(dev) for _ in range(2)]
        # undivided reference on this GPU
        km = pce.KernelMap(torch.from_numpy(coords_h).to(dev), (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
        ref = feats_all.to(dev)
        for w in ws:
            ref = PF.conv_forward(ref, w, km.csr(), PF.FusedEpilogue(act="relu"))
        # two slabs, halo pushed by the epilogue
        cuts, owned = mg.split_scene(coords_h, world, radius)
        idx = owned[rank]
        scene = mg.SlabScene(torch.from_numpy(coords_h[idx]).to(dev), cuts, rank, world, radius).setup()
        push = mg.PeerPush(scene, c, torch.float16)
        push.owned(0).copy_(feats_all[idx].to(dev))
        scene.exchange_into(push.local(0))
        lkm = pce.KernelMap(scene.local_coords, (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
        csr = lkm.csr().restrict(scene.n_owned)
        for i, w in enumerate(ws):
            src, dst = i & 1, (i & 1) ^ 1
            PF.conv_forward(push.local(src), w, csr, push.epilogue(dst, act="relu"), out=push.owned(dst))
            push.barrier(dst)
        torch.cuda.synchronize()
        got = push.owned(0)
        ok = bool(torch.equal(got, ref[torch.from_numpy(idx).to(dev)])) and PF.device_status() == 0
        # the halo rows of the last written buffer hold the neighbours' boundary rows of that layer
        nl = int(scene.halo_left.size(0))
        halo = push.local(0)[scene.n_owned:]
        halo_idx = []
        lut = {tuple(r): i for i, r in enumerate(coords_h.tolist())}
        for r in scene.local_coords[scene.n_owned:].cpu().tolist():
            halo_idx.append(lut[tuple(r)])
        ok = ok and bool(torch.equal(halo, ref[torch.tensor(halo_idx, device=dev)])) and halo.size(0) > 0 and nl >= 0
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_halo_pushed_by_the_epilogue_matches_the_undivided_scene():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert ret.get(0) is True and ret.get(1) is True
