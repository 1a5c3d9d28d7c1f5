"""Whole-network parity: the MinkUNet-shaped model on the GPU against its CPU restatement."""
import numpy as np
import pytest
import torch

from oracle import conv_oracle as co
from oracle import minkunet_oracle as mo
from tests.helpers import cmax_of, surface_cloud

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 5e-3)])
def test_minkunet_matches_oracle(dtype, tol):
    import pcengine_b200 as pce
    coords = surface_cloud(31, 64, batch=2)
    torch.manual_seed(7)
    feats = torch.randn(len(coords), 4).to(dtype)
    model = pce.MinkUNet(4, 19, cr=0.5)
    pce.randomize_batchnorm(model, 3)
    model = model.to(dtype).eval()
    ref = mo.forward(model.state_dict(), coords, feats, act_dtype=dtype)
    model = model.cuda()
    x = pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords),
                     init_tag=pce.MinkUNet.tags())
    with torch.no_grad():
        y = model(x)
    assert y.feats.shape == (len(coords), 19) and y.coords.data_ptr() == x.coords.data_ptr()
    assert len(y.kmaps) == 9
    assert co.rel_l2(y.feats.float().cpu(), ref) <= tol


def test_fused_and_module_paths_agree():
    """Eval-mode fusion gives the same numbers as running conv, BatchNorm and ReLU one by one."""
    import pcengine_b200 as pce
    from pcengine_b200.minkunet import ConvBNReLU, ResidualBlock
    coords = surface_cloud(5, 40)
    torch.manual_seed(1)
    feats = torch.randn(len(coords), 16)

    def tensor():
        return pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords),
                            init_tag=["auto"])
    for block in (ConvBNReLU(16, 32), ResidualBlock(16, 32), ResidualBlock(16, 16)):
        pce.randomize_batchnorm(block, 2)
        block = block.cuda().eval()
        with torch.no_grad():
            fused = block(tensor()).feats
            block._fused = lambda x: False
            plain = block(tensor()).feats
        assert co.rel_l2(fused.cpu(), plain.cpu()) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_planned_maps_equal_lazy_maps(dtype):
    """The planning thread leaves the same maps in the tensor (coordinates, map table, offsets, CSR,
    tile lists) and the same logits, bit for bit, as building each map at the layer that first needs
    it; repeated passes recycle the planner's storage."""
    import pcengine_b200 as pce
    coords = surface_cloud(44, 72, batch=3)
    torch.manual_seed(11)
    feats = torch.randn(len(coords), 4).to(dtype)
    model = pce.MinkUNet(4, 19, cr=0.5)
    pce.randomize_batchnorm(model, 5)
    model = model.to(dtype).eval().cuda()

    def run(plan_ahead):
        model.plan_ahead = plan_ahead
        x = pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords),
                         init_tag=["auto"])
        with torch.no_grad():
            y = model(x)
        torch.cuda.synchronize()
        return y
    lazy, planned = run(False), run(True)
    for _ in range(3):
        planned = run(True)
    assert type(next(iter(planned.kmaps.values()))).__name__ == "PlannedKernelMap"
    assert torch.equal(lazy.feats, planned.feats)
    assert sorted(lazy.kmaps) == sorted(planned.kmaps) and len(planned.kmaps) == 9
    for key, a in lazy.kmaps.items():
        b = planned.kmaps[key]
        assert (a.n_in, a.n_out, a.kv, a.symmetric) == (b.n_in, b.n_out, b.kv, b.symmetric)
        assert torch.equal(a.out_coords, b.out_coords) and torch.equal(a.map, b.map.tensor())
        assert torch.equal(a.kpos, b.kpos.tensor()) and torch.equal(a.qkpos, b.qkpos.tensor())
        assert a.sizes() == b.sizes()
        for tr, ca in a._csr.items():
            cb = b._csr[tr]
            p = int(ca.rowptr[-1])
            # (a planned map that only needed tile lists builds rowptr / nbr on this first access)
            as_tensor = lambda v: v if isinstance(v, torch.Tensor) else v.tensor()
            assert torch.equal(ca.mask, cb.mask.tensor()) and torch.equal(ca.rowptr, as_tensor(cb.rowptr))
            assert torch.equal(ca.nbr[:p], as_tensor(cb.nbr)[:p])
            assert bool(cb._tiles) == (dtype == torch.float16)  # tile lists feed the tensor-core kernel only
            for tk, tb in cb._tiles.items():
                ca.tiles(*tk)
                ta = ca._tiles[tk]
                stages = int(ta[2][-1])
                assert torch.equal(ta[1], tb[1].tensor()) and torch.equal(ta[2], tb[2].tensor())
                assert torch.equal(ta[3][:stages], tb[3].tensor()[:stages])
                assert torch.equal(ta[4][:stages * tk[1]], tb[4].tensor()[:stages * tk[1]])


def test_map_plan_api():
    """MapPlan on a hand-written layer list: maps not in the plan are still built lazily, a tensor the
    plan does not fit stays on the lazy path, and the reference forms derive from a planned map."""
    import pcengine_b200 as pce
    coords = surface_cloud(45, 48)
    cm = cmax_of(coords)

    def tensor():
        return pce.spTensor(torch.randn(len(coords), 16, generator=torch.Generator().manual_seed(3)).half().cuda(),
                            torch.from_numpy(coords).cuda(), None, [0, 0, 0], cm, init_tag=["auto"])
    plan = pce.MapPlan([(3, 1, False, 16, 32), (2, 2, False, 32, 32), (3, 1, False, 32, 64), (2, 2, True, 64, 32)])
    with pytest.raises(RuntimeError):
        pce.MapPlan([(2, 2, True, 64, 32)])
    conv = pce.conv3d(16, 32, 3).cuda().half()
    down = pce.conv3d(32, 32, 2, 2).cuda().half()
    five = pce.conv3d(32, 32, 5).cuda().half()
    up = pce.conv3d(32, 16, 2, 2, transposed=True).cuda().half()
    outs = []
    for planned in (False, True):
        x = tensor()
        assert plan.begin(x) if planned else True
        a = conv(x)
        b = down(a)
        c = five(b)          # 5x5x5 at the coarse level is not in the plan
        d = up(c)
        outs.append((a.feats, b.feats, c.feats, d.feats, b.coords, d.coords))
        if planned:
            km = x.kmaps[(conv.kernel_size_code, x.stride, conv.stride_code)]
            lazy_km = pce.KernelMap(x.coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cm, True)
            for got, want in zip(km.pairs(), lazy_km.pairs()):
                assert torch.equal(got, want)
            for got, want in zip(km.d1(), lazy_km.d1()):
                assert torch.equal(got, want)
    for u, v in zip(*outs):
        assert torch.equal(u, v)
    x = tensor()
    x.stride = pce.conv_info_encoder([2, 2, 2])
    assert plan.begin(x) is False and x.planner is None
    plan.close()
    assert plan.begin(tensor()) is False


def test_planned_pass_on_a_side_stream():
    """The network run on a stream of its own, with the coordinates produced on yet another one
    (``coords_ready``), gives the logits of the plain run; storage released from that stream is
    recycled safely over repeated passes."""
    import pcengine_b200 as pce
    coords = surface_cloud(46, 64, batch=2)
    torch.manual_seed(12)
    feats = torch.randn(len(coords), 4).half().cuda()
    model = pce.MinkUNet(4, 19, cr=0.5)
    pce.randomize_batchnorm(model, 6)
    model = model.half().eval().cuda()
    cm = cmax_of(coords)
    coords_pin = torch.from_numpy(coords).pin_memory()
    with torch.no_grad():
        want = model(pce.spTensor(feats, coords_pin.cuda(), None, [0, 0, 0], cm, init_tag=["auto"])).feats.clone()
    torch.cuda.synchronize()
    work, copy = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(6):
        with torch.cuda.stream(copy):
            c = coords_pin.to("cuda", non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(copy)
        work.wait_event(ready)
        with torch.cuda.stream(work), torch.no_grad():
            x = pce.spTensor(feats, c, None, [0, 0, 0], cm, init_tag=["auto"])
            x.coords_ready = ready
            got = model(x).feats
            c.record_stream(work)
        del x
    work.synchronize()
    assert torch.equal(got, want)


def test_many_live_passes_fall_back_to_lazy_maps():
    """Keeping the outputs (and with them the planner storage) of more passes than the planner holds
    arenas for makes further passes build their maps lazily; every result stays the same."""
    import pcengine_b200 as pce
    coords = surface_cloud(47, 40)
    torch.manual_seed(13)
    feats = torch.randn(len(coords), 4).half().cuda()
    model = pce.MinkUNet(4, 19, cr=0.25)
    pce.randomize_batchnorm(model, 7)
    model = model.half().eval().cuda()
    kept = []
    for _ in range(11):
        x = pce.spTensor(feats, torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords), init_tag=["auto"])
        with torch.no_grad():
            kept.append(model(x))
    kinds = [type(next(iter(y.kmaps.values()))).__name__ for y in kept]
    assert kinds[:8] == ["PlannedKernelMap"] * 8 and kinds[8:] == ["KernelMap"] * 3
    for y in kept[1:]:
        assert torch.equal(y.feats, kept[0].feats)
    del kept, y
    x = pce.spTensor(feats, torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords), init_tag=["auto"])
    with torch.no_grad():
        again = model(x)
    assert type(next(iter(again.kmaps.values()))).__name__ == "PlannedKernelMap"  # storage came back


@pytest.mark.parametrize("n", [0, 1, 5])
def test_network_on_nearly_nothing(n):
    """The whole network (planner path included) on zero, one and five voxels: shapes hold and the
    planned run equals the lazy one."""
    import pcengine_b200 as pce
    coords = np.array([[0, 3, 3, 3], [0, 3, 3, 4], [0, 20, 20, 20], [1, 3, 3, 3], [1, 40, 2, 9]], np.int32)[:n].reshape(-1, 4)
    torch.manual_seed(14)
    feats = torch.randn(n, 4).half().cuda()
    model = pce.MinkUNet(4, 19, cr=0.25)
    pce.randomize_batchnorm(model, 8)
    model = model.half().eval().cuda()
    outs = []
    for plan in (True, False):
        model.plan_ahead = plan
        x = pce.spTensor(feats, torch.from_numpy(coords).cuda(), None, [0, 0, 0], [63, 63, 63], init_tag=["auto"])
        with torch.no_grad():
            outs.append(model(x).feats)
    assert outs[0].shape == (n, 19) and torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("cr", [1.0, 0.5, 0.3])
def test_shared_skip_buffers_equal_concatenation(cr):
    """fp16 inference writes every decoder input [up-sampled | skip] as one matrix (the skip layer and the
    up-sampling layer each write their column range); the logits are the bits of the path that
    concatenates.  cr = 0.3 gives widths the kernel cannot address in place (copies take over)."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(41, 72, batch=3)
    torch.manual_seed(11)
    feats = torch.randn(len(coords), 4).half()
    model = pce.MinkUNet(4, 19, cr=cr)
    pce.randomize_batchnorm(model, 5)
    model = model.half().eval().cuda()

    def run():
        x = pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords), batchsize=3,
                         init_tag=pce.MinkUNet.tags())
        with torch.no_grad():
            return model(x).feats
    assert model.shared_skip_buffers
    shared = run()
    model.shared_skip_buffers = False
    joined = run()
    assert torch.equal(shared, joined)
    assert PF.device_status() == 0


def test_plan_before_forward():
    """MinkUNet.plan(x) starts the map construction ahead of forward(x): same logits, a second call
    is a no-op, and passes that were planned and never run are given back."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(51, 72, batch=2)
    torch.manual_seed(3)
    feats = torch.randn(len(coords), 4).half()
    model = pce.MinkUNet(4, 19, cr=0.5)
    pce.randomize_batchnorm(model, 9)
    model = model.half().eval().cuda()

    def tensor():
        return pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords), batchsize=2,
                            init_tag=pce.MinkUNet.tags())
    with torch.no_grad():
        want = model(tensor()).feats
        for _ in range(12):  # more than the planner keeps passes for: dropped passes must come back
            x = tensor()
            assert model.plan(x)
            del x
        a, b = tensor(), tensor()
        assert model.plan(a) and model.plan(b) and not model.plan(a)
        assert a.planner is not None and b.planner is not None
        got_b = model(b).feats  # out of order on purpose
        got_a = model(a).feats
    assert torch.equal(got_a, want) and torch.equal(got_b, want)
    model.train()
    assert not model.plan(tensor())
    assert PF.device_status() == 0


def test_one_call_pass_equals_the_layer_by_layer_pass():
    """The whole pass as one library call (NetProgram / pce_net_run) issues the launches of the
    layer-by-layer path: logits bit-identical, the tensor's kernel maps there when asked for, passes
    recycled run after run, and a change of the weights is picked up after invalidate_packed."""
    import pcengine_b200 as pce
    coords = surface_cloud(61, 72, batch=3)
    torch.manual_seed(3)
    feats = torch.randn(len(coords), 4).half()
    model = pce.MinkUNet(4, 19, cr=1.0)
    pce.randomize_batchnorm(model, 5)
    model = model.half().eval().cuda()

    def tensor():
        return pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords), batchsize=3,
                            init_tag=pce.MinkUNet.tags())

    with torch.no_grad():
        model.one_call = False
        want = model(tensor())
        model.one_call = True
        for _ in range(6):  # more passes than the planner keeps arenas for
            x = tensor()
            got = model(x)
            assert torch.equal(got.feats, want.feats)
        assert model.__dict__["_programs"] and all(p is not None for p in model.__dict__["_programs"].values())
        assert len(got.kmaps) == 9 == len(want.kmaps)
        for key, km in want.kmaps.items():
            assert torch.equal(got.kmaps[key].map.tensor(), km.map.tensor())
            assert torch.equal(got.kmaps[key].out_coords, km.out_coords)
        ref = mo.forward(model.state_dict(), coords, feats)
        assert co.rel_l2(got.feats.float().cpu(), ref) <= 5e-3
        # new weights: both paths follow after the cached layouts are dropped
        model.stem[1].conv.kernel.data.mul_(0.5)
        pce.invalidate_packed(model)
        model.one_call = False
        want2 = model(tensor())
        model.one_call = True
        got2 = model(tensor())
        assert torch.equal(got2.feats, want2.feats) and not torch.equal(got2.feats, want.feats)
    from pcengine_b200 import functional as PF
    assert PF.device_status() == 0


def test_planner_routes_build_the_same_lists():
    """A planned map of at most 32 offsets whose layers all run on tile lists arrives without rowptr / nbr
    (the lists were filled straight from the dense table, the row order came from knnz): its bitmask, row order
    and tile lists are those of the route through the neighbour CSR (pce_tune(9, 0)), the logits are the same
    bit for bit, and rowptr / nbr appear, equal to the other route's, when they are first asked for."""
    import pcengine_b200 as pce
    from pcengine_b200 import _lib
    coords = surface_cloud(46, 72, batch=2)
    torch.manual_seed(12)
    feats = torch.randn(len(coords), 4).half()
    model = pce.MinkUNet(4, 19, cr=0.5)
    pce.randomize_batchnorm(model, 6)
    model = model.half().eval().cuda()

    def run(short):
        assert _lib.lib.pce_tune(9, short) == 0
        x = pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords), batchsize=2,
                         init_tag=pce.MinkUNet.tags())
        with torch.no_grad():
            y = model(x)
        torch.cuda.synchronize()
        return y
    try:
        run(1)
        through_csr, short = run(0), run(1)
    finally:
        _lib.lib.pce_tune(9, 1)
    assert torch.equal(through_csr.feats, short.feats)
    assert len(short.kmaps) == 9
    skipped = 0
    for key, a in through_csr.kmaps.items():
        b = short.kmaps[key]
        assert type(b).__name__ == "PlannedKernelMap"
        for tr, ca in a._csr.items():
            cb = b._csr[tr]
            assert ca._rowptr is not None and ca._fill is None
            skipped += cb._rowptr is None
            assert torch.equal(ca.mask.tensor(), cb.mask.tensor())
            assert sorted(ca._tiles) == sorted(cb._tiles) and cb._tiles
            for tk, ta in ca._tiles.items():
                tb = cb._tiles[tk]
                stages = int(ta[2].tensor()[-1])
                assert torch.equal(ta[1].tensor(), tb[1].tensor()) and torch.equal(ta[2].tensor(), tb[2].tensor())
                assert torch.equal(ta[3].tensor()[:stages], tb[3].tensor()[:stages])
                assert torch.equal(ta[4].tensor()[:stages * tk[1]], tb[4].tensor()[:stages * tk[1]])
            p = int(ca.rowptr.tensor()[-1])
            assert cb._rowptr is None and int(cb.pair_count()) == p == int(ca.pair_count())  # (from knnz, nothing built)
            assert torch.equal(ca.rowptr.tensor(), cb.rowptr if isinstance(cb.rowptr, torch.Tensor) else cb.rowptr.tensor())
            got_nbr = cb.nbr if isinstance(cb.nbr, torch.Tensor) else cb.nbr.tensor()
            assert torch.equal(ca.nbr.tensor()[:p], got_nbr[:p])
            assert cb._rowptr is not None and cb._fill is None
    total = sum(len(a._csr) for a in through_csr.kmaps.values())
    assert skipped == total == 13  # five submanifold maps (one direction each) and four strided ones (two each)


def test_planned_map_with_more_than_32_offsets_keeps_its_csr():
    """A 5x5x5 layer in a plan (125 offsets: two-word sort keys) goes through the neighbour CSR inside the
    planner, a 3x3x3 layer of the same plan does not; both give the lazy path's results bit for bit."""
    import pcengine_b200 as pce
    coords = surface_cloud(47, 40)
    cm = cmax_of(coords)
    feats = torch.randn(len(coords), 32, generator=torch.Generator().manual_seed(4)).half()

    def tensor():
        return pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], cm, init_tag=["auto"])
    three = pce.conv3d(32, 32, 3).cuda().half()
    five = pce.conv3d(32, 64, 5).cuda().half()
    plan = pce.MapPlan([(3, 1, False, 32, 32), (5, 1, False, 32, 64)])
    outs = []
    for planned in (False, True):
        x = tensor()
        assert plan.begin(x) if planned else True
        with torch.no_grad():
            a = three(x)
            b = five(a)
        outs.append((a.feats, b.feats))
        if planned:
            k3 = x.kmaps[(three.kernel_size_code, x.stride, three.stride_code)]
            k5 = x.kmaps[(five.kernel_size_code, x.stride, five.stride_code)]
            assert type(k5).__name__ == "PlannedKernelMap" and k5.kv == 125
            assert k3._csr[False]._rowptr is None and k5._csr[False]._rowptr is not None
    torch.cuda.synchronize()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    plan.close()
