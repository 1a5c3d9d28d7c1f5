"""Two things on a scene cut into two slabs, one per GPU.  (1) A U-shaped chain of layers (3x3x3, 2x2x2 stride 2 down, 3x3x3, transposed 2x2x2 up, 3x3x3) on a scene cut
into two slabs whose planes are multiples of the stride, one slab per GPU: the down- and up-sampling layers run
on owned rows with no exchange, the submanifold layers exchange their level's halo (NCCL point-to-point), and
the owned rows of both slabs equal the undivided scene computed on one GPU.  (2) The MinkUNet module itself on
``spTensor.slabs`` (four down-sampling levels, cuts at multiples of 16): conv_func exchanges every submanifold
layer's halo, and each rank's logits are the undivided network's logits for its voxels.  Needs two GPUs; skipped
otherwise."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    import pcengine_b200 as pce
    from oracle import conv_oracle as co
    from pcengine_b200 import functional as PF, multigpu as mg, synth
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        xyz, _ = synth.indoor_room(3002, 60000)
        coords_h = synth.with_batch(xyz)
        cmax = coords_h[:, 1:].max(0).tolist()
        g = torch.Generator().manual_seed(7)
        c0, c1 = 32, 64
        feats_all = torch.randn(len(coords_h), c0, generator=g).half()

        def weight(kv, cin, cout):
            return (torch.randn(kv, cin, cout, generator=g) / (kv * cin) ** 0.5).half().to(dev)
        w0, wd, w1, wu, w2 = weight(27, c0, c0), weight(8, c0, c1), weight(27, c1, c1), weight(8, c1, c0), weight(27, c0, c0)
        relu = PF.FusedEpilogue(act="relu")
        sub, down, z = ((3, 3, 3), (1, 1, 1)), ((2, 2, 2), (2, 2, 2)), (0, 0, 0)

        def chain(x, m0, md, m1, n0=None, n1=None, ex0=None, ex1=None):
            """The five layers; n0 / n1 restrict the submanifold layers to the owned rows and ex0 / ex1 turn owned
            rows into [owned | halo] rows (slab run); all None for the undivided scene."""
            csr0 = m0.csr() if n0 is None else m0.csr().restrict(n0)
            csr1 = m1.csr() if n1 is None else m1.csr().restrict(n1)
            grow0 = ex0 or (lambda t: t)
            grow1 = ex1 or (lambda t: t)
            a = PF.conv_forward(grow0(x), w0, csr0, relu)
            b = PF.conv_forward(a, wd, md.csr(), relu)
            c = PF.conv_forward(grow1(b), w1, csr1, relu)
            u = PF.conv_forward(c, wu, md.csr(transposed=True), relu)
            return b, PF.conv_forward(grow0(u), w2, csr0)
        # the undivided scene on this GPU
        full = torch.from_numpy(coords_h).to(dev)
        f0 = pce.KernelMap(full, *sub, z, [0, 0, 0], cmax, True)
        cmax1 = mg.coarse_bounds(cmax, 2)
        fd = pce.KernelMap(full, *down, z, [0, 0, 0], cmax1, False)
        fd.build()
        f1 = pce.KernelMap(fd.out_coords, *sub, z, [0, 0, 0], cmax1, True)
        ref_b, ref_y = chain(feats_all.to(dev), f0, fd, f1)
        # two slabs with even cut planes
        cuts, owned = mg.split_scene(coords_h, world, 1, align=2)
        idx = owned[rank]
        levels = mg.SlabLevels(torch.from_numpy(coords_h[idx]).to(dev), cuts, rank, world, 1, [2], cmax)
        s0, s1 = levels[0], levels[1]
        m0 = pce.KernelMap(s0.local_coords, *sub, z, [0, 0, 0], cmax, True)
        md = pce.KernelMap(s0.coords, *down, z, [0, 0, 0], levels.cmax[1], False)   # owned rows only: no halo
        md.build()
        m1 = pce.KernelMap(s1.local_coords, *sub, z, [0, 0, 0], levels.cmax[1], True)
        ok = bool(torch.equal(md.out_coords, s1.coords)) and levels.cmax[1] == cmax1
        got_b, got_y = chain(feats_all[idx].to(dev), m0, md, m1, s0.n_owned, s1.n_owned, s0.local_feats, s1.local_feats)
        torch.cuda.synchronize()
        lut = {tuple(r): i for i, r in enumerate(fd.out_coords.cpu().tolist())}
        idx1 = torch.tensor([lut[tuple(r)] for r in s1.coords.cpu().tolist()], device=dev)
        err_b = co.rel_l2(got_b.float().cpu(), ref_b[idx1].float().cpu())
        err_y = co.rel_l2(got_y.float().cpu(), ref_y[torch.from_numpy(idx).to(dev)].float().cpu())
        counts = [None] * world
        dist.all_gather_object(counts, s1.n_owned)
        ok = ok and sum(counts) == fd.n_out and s1.halo_left.size(0) + s1.halo_right.size(0) > 0
        # (2) the whole network
        model = pce.MinkUNet(4, 19, cr=0.5)
        pce.randomize_batchnorm(model, 8)
        model = model.half().eval().to(dev)
        feats4 = torch.randn(len(coords_h), 4, generator=g).half()
        with torch.no_grad():
            whole = model(pce.spTensor(feats4.to(dev), full, None, [0, 0, 0], cmax, init_tag=pce.MinkUNet.tags())).feats
            cuts16, owned16 = mg.split_scene(coords_h, world, 1, align=16)
            mine = owned16[rank]
            x = pce.spTensor(feats4[mine].to(dev), torch.from_numpy(coords_h[mine]).to(dev), None, [0, 0, 0], cmax,
                             init_tag=pce.MinkUNet.tags())
            x.slabs = mg.SlabLevels(x.coords, cuts16, rank, world, 1, [2, 2, 2, 2], cmax)
            part = model(x)
        torch.cuda.synchronize()
        err_net = co.rel_l2(part.feats.float().cpu(), whole[torch.from_numpy(mine).to(dev)].float().cpu())
        ok = ok and part.slabs is x.slabs and part.feats.shape == (len(mine), 19) and x.planner is None
        ok = ok and any(isinstance(k, tuple) and k[0] == "slab" for k in part.kmaps)
        # the halo rows went through symmetric-memory mailboxes (peer stores), not messages, wherever a row is a
        # multiple of 16 bytes; the same pass with messages throughout gives the same logits bit for bit
        boxes = x.slabs.__dict__.get("_mailboxes", {})
        ok = ok and len(boxes) > 0 and all(v is not None for v in boxes.values())
        with torch.no_grad():
            x2 = pce.spTensor(feats4[mine].to(dev), torch.from_numpy(coords_h[mine]).to(dev), None, [0, 0, 0], cmax,
                              init_tag=pce.MinkUNet.tags())
            x2.slabs = x.slabs
            x2.slabs.use_mailboxes = False
            ok = ok and bool(torch.equal(model(x2).feats, part.feats))
            x2.slabs.use_mailboxes = True
        ret[rank] = (ok and err_b <= 1e-3 and err_y <= 1e-3 and err_net <= 2e-3 and PF.device_status() == 0,
                     err_b, err_y, err_net)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_layers_and_network_on_two_slabs_match_the_undivided_scene():
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
    assert ret.get(0) is not None and ret.get(1) is not None
    assert ret[0][0] is True and ret[1][0] is True, (ret[0], ret[1])
