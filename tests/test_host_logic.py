"""Host-side pieces of the operator surface that need no GPU."""
import numpy as np
import pytest
import torch

import pcengine_b200 as pce
from oracle import kmap_oracle as ko
from pcengine_b200 import synth


def test_codes_round_trip_and_stride_composition():
    for v in ([1, 1, 1], [3, 3, 3], [2, 1, 5], [0, 0, 0]):
        assert list(pce.conv_info_decoder(pce.conv_info_encoder(v))) == v
        assert pce.conv_info_encoder(v) == ko.encode3(v)
    assert pce.conv_info_encoder([1, 1, 1]) == 94585  # default tensor stride of spTensor
    s2 = pce.conv_info_encoder([2, 2, 2])
    s4 = pce.output_stride_compute(s2, s2, 0)
    assert pce.conv_info_decoder(s4) == (4, 4, 4)
    assert pce.output_stride_compute(s2, s4, 1) == s2


def test_sptensor_surface():
    feats = torch.randn(5, 3)
    coords = torch.tensor([[0, 1, 2, 3]] * 5, dtype=torch.int32)
    x = pce.spTensor(feats, coords, None, [0, 0, 0], [1, 2, 3])
    assert x.stride == 94585 and x.init_tag == ["end"] and x.batchsize == 1
    assert x.F is feats and x.C is coords and pce.SparseTensor is pce.spTensor
    y = x + x
    assert torch.equal(y.feats, feats * 2) and y.kmaps is x.kmaps and y.cbook is x.cbook
    z = pce.cat([x, y])
    assert z.feats.shape == (5, 6)
    r = pce.ReLU()(x)
    assert (r.feats >= 0).all() and r.coords is coords
    bn = pce.BatchNorm(3).eval()
    assert pce.BatchNorm.__mro__[1] is torch.nn.BatchNorm1d
    out = bn(x)  # CPU tensors go through nn.BatchNorm1d itself
    assert out.feats.shape == (5, 3)
    x.build_buffer({"in": [4], "out": [8], "kernel": [3]}, "cpu")
    assert x.buffer.numel() == 12 * 5 * 16


def test_conv3d_parameters_match_reference_layout():
    c = pce.conv3d(8, 16, 3, 1, bias=True)
    assert c.kernel.shape == (27, 8, 16) and c.bias.shape == (16,)
    bound = 1.0 / (16 * 27) ** 0.5
    assert float(c.kernel.abs().max()) <= bound
    assert pce.conv3d(8, 16, 1).kernel.shape == (8, 16)
    assert pce.conv3d(4, 4, [3, 1, 5]).kernel_volume == 15
    assert "transposed=True" in repr(pce.conv3d(4, 4, 2, 2, transposed=True))
    assert set(c.state_dict().keys()) == {"kernel", "bias"}


def test_quantize_and_collate():
    rng = np.random.default_rng(0)
    pts = rng.uniform(0, 4, (2000, 3))
    v, idx, inv = pce.sparse_quantize(pts, 0.5, return_index=True, return_inverse=True)
    assert len(np.unique(v, axis=0)) == len(v) and (v[inv] == np.floor(pts / 0.5).astype(np.int32)).all()
    a = pce.spTensor(torch.randn(len(v), 2), torch.from_numpy(v), None, [0, 0, 0], v.max(0).tolist(), init_tag=["D2", "end"])
    b = pce.spTensor(torch.randn(len(v), 2), torch.from_numpy(v), None, [0, 0, 0], v.max(0).tolist())
    c = pce.sparse_collate([a, b])
    assert c.coords.shape == (2 * len(v), 4) and c.batchsize == 2 and c.init_tag == ["D2", "end"]
    assert c.coords[:, 0].unique().tolist() == [0, 1]
    out = pce.sparse_collate_fn([{"x": a, "y": np.zeros(3)}, {"x": b, "y": np.ones(3)}])
    assert out["x"].batchsize == 2 and out["y"].shape == (6,)


def test_layer_scheduler():
    assert pce.init_layer_scheduler({"stride": [1, 1, 2], "in": [4, 32, 32], "out": [32, 32, 64]}) == "simple"
    assert pce.init_layer_scheduler({"stride": [1, 1, 2], "in": [4, 64, 64], "out": [64, 64, 64]}) == "whole"


def test_generators_are_seeded_and_unique():
    a = synth.uniform_grid(20000, 64, 1001)
    assert a.shape == (20000, 3) and len(np.unique(a, axis=0)) == 20000 and a.max() < 64
    assert np.array_equal(a, synth.uniform_grid(20000, 64, 1001))
    s = synth.lidar_scan(2000)
    assert 40000 < len(s) < 130000 and s.min() == 0 and len(np.unique(s, axis=0)) == len(s)
    r, m = synth.indoor_room(3001, 20000)
    assert abs(len(r) - 20000) <= 600


def test_map_plan_specs_of_the_unet():
    """MapPlan turns the network's layer list into map specs in first-use order: five submanifold maps,
    four strided ones (each opening a coordinate level), transposed layers folded into their strided
    map, widths rounded up to the tensor-core granule."""
    model = pce.MinkUNet(4, 19)
    plan = pce.MapPlan(model.layer_plan())
    assert len(plan.specs) == 9 and plan.n_levels == 4
    assert [s["subm"] for s in plan.specs] == [True, False, True, False, True, False, True, False, True]
    assert [s["in_level"] for s in plan.specs] == [0, 0, 1, 1, 2, 2, 3, 3, 4]
    assert [s["out_level"] for s in plan.specs] == [0, 1, 1, 2, 2, 3, 3, 4, 4]
    # uses are (C_out, C_in) rounded up to the tensor-core granule: the 4-channel stem reads 16
    assert plan.specs[0]["fwd"] == [(32, 16), (32, 32), (96, 128), (96, 96)] and plan.specs[0]["tr"] == []
    assert plan.specs[1]["fwd"] == [(32, 32)] and plan.specs[1]["tr"] == [(96, 96)]
    assert plan.specs[8]["fwd"] == [(256, 128), (256, 256)]
    c = plan._c_specs()
    assert c[1].want_fwd == 1 and c[1].want_tr == 1 and list(c[1].c_out_tr)[:2] == [96, 0]
    assert list(c[0].c_in_fwd)[:4] == [16, 32, 128, 96]
    assert list(c[0].ks) == [3, 3, 3] and list(c[1].stride) == [2, 2, 2] and c[3].in_level == 1
    ragged = pce.MapPlan([(3, 1, False, 4, 19)], dtype=torch.float32)
    assert ragged.specs[0]["fwd"] == [(32, 16)] and list(ragged._c_specs()[0].c_out_fwd)[:1] == [0]  # no tile lists for fp32
    import pytest
    with pytest.raises(ValueError):
        pce.MapPlan([(1, 1, False, 8, 8)])


def test_nothing_is_planned_for_cpu_tensors_or_in_training():
    """MinkUNet.plan starts a map construction only for CUDA tensors in eval mode; anything else is
    left to the layers (which refuse CPU tensors themselves)."""
    import torch

    import pcengine_b200 as pce
    coords = torch.zeros((8, 4), dtype=torch.int32)
    coords[:, 1] = torch.arange(8, dtype=torch.int32)
    x = pce.spTensor(torch.zeros(8, 4), coords, None, [0, 0, 0], [7, 0, 0], init_tag=pce.MinkUNet.tags())
    model = pce.MinkUNet(4, 19, cr=0.25).eval()
    assert model.plan(x) is False and x.planner is None
    model.train()
    assert model.plan(x) is False
    model.plan_ahead = False
    model.eval()
    assert model.plan(x) is False


def test_row_pitched_views():
    """Which feature matrices the tensor-core kernel may address in place: fp16, rows contiguous, pitch a
    multiple of 8 elements, 16-byte aligned start."""
    import torch

    from pcengine_b200.functional import _row_pitched
    wide = torch.zeros((10, 64), dtype=torch.float16)
    assert _row_pitched(wide) and _row_pitched(wide[:, 8:40]) and _row_pitched(wide[:, 16:])
    assert not _row_pitched(wide[:, 3:35])          # start not 16-byte aligned
    assert not _row_pitched(wide.t())               # rows not contiguous
    assert not _row_pitched(torch.zeros((10, 12), dtype=torch.float16))  # pitch 12 is no multiple of 8
    assert not _row_pitched(wide.float()[:, 8:40])  # fp32 goes through the CUDA-core kernel


def test_dataflow_selector_follows_the_measured_table():
    """'auto' picks the explicit gather-GEMM-scatter dataflow only where the sweep measured it faster
    (wide fp16 layers on small, very sparse maps); tags 'D1' / 'D2' are taken as given; the sparsity
    callable is evaluated only when width and map size already qualify."""
    import torch
    from pcengine_b200.spconv import _choose_dataflow
    assert _choose_dataflow("D1", 16, 16) == "D1" and _choose_dataflow("D2", 256, 256, 1.0, 1000, torch.float16) == "D2"
    assert _choose_dataflow("auto", 256, 256, 1.2, 25000, torch.float16) == "D1"
    assert _choose_dataflow("auto", 256, 256, 2.7, 25000, torch.float16) == "D2"     # denser neighbourhoods
    assert _choose_dataflow("auto", 256, 256, 1.2, 200000, torch.float16) == "D2"    # large map
    assert _choose_dataflow("auto", 128, 256, 1.2, 25000, torch.float16) == "D2"     # narrower input
    assert _choose_dataflow("auto", 256, 256, 1.2, 25000, torch.float32) == "D2"     # fp32 runs on CUDA cores
    assert _choose_dataflow("auto", 256, 256) == "D2"                                # facts missing

    def never():
        raise AssertionError("sparsity was read although width / size rule the explicit dataflow out")
    assert _choose_dataflow("auto", 64, 64, never, 25000, torch.float16) == "D2"
    assert _choose_dataflow("auto", 256, 256, never, 10 ** 6, torch.float16) == "D2"


def test_neighbour_csr_builds_missing_arrays_once():
    """A CSR that arrives without rowptr / nbr (a planned map whose tile lists came straight from the dense
    table) asks its `fill` for them on first use, once, and keeps the result; a complete one never does."""
    from pcengine_b200.kmap import NeighbourCSR
    calls = []
    rowptr, nbr = torch.tensor([0, 2, 3], dtype=torch.int32), torch.tensor([1, 0, 1], dtype=torch.int32)

    def fill():
        calls.append(1)
        return rowptr, nbr
    mask = torch.tensor([[3], [2]], dtype=torch.int32)
    lazy = NeighbourCSR(mask, None, None, 2, 2, kv=2, fill=fill)
    assert lazy._rowptr is None and not calls
    assert lazy.nbr is nbr and lazy.rowptr is rowptr and lazy.rowptr is rowptr and len(calls) == 1
    assert lazy.restrict(1).rowptr.tolist() == [0, 2]
    whole = NeighbourCSR(mask, rowptr, nbr, 2, 2, kv=2, fill=fill)
    assert whole.rowptr is rowptr and len(calls) == 1


def test_slab_tensors_refuse_layers_that_would_need_rows_across_a_cut():
    """On a tensor that holds one rank's slab of a scene, a down-sampling layer must have kernel size == stride
    and no padding (its inputs then all lie in the slab): anything else is refused before any kernel runs, and
    the marker travels with the tensor through the feature-wise operators."""
    from pcengine_b200 import multigpu as mg
    coords = synth.with_batch(synth.uniform_grid(500, 16, seed=3))
    cmax = coords[:, 1:].max(0).tolist()
    x = pce.spTensor(torch.randn(len(coords), 8), torch.from_numpy(coords), None, [0, 0, 0], cmax, init_tag=["auto"])
    x.slabs = mg.SlabLevels(x.coords, [0, 16], 0, 1, 1, [2], cmax)
    assert pce.ReLU()(x).slabs is x.slabs and pce.cat([x, x]).slabs is x.slabs and (x + x).slabs is x.slabs
    with pytest.raises(NotImplementedError, match="kernel size == stride"):
        pce.conv3d(8, 8, 3, 2)(x)
    with pytest.raises(NotImplementedError, match="kernel size == stride"):
        pce.conv3d(8, 8, 2, 2, padding=1)(x)
    assert x.slabs.level_of([2, 2, 2]) == 1
