"""Parity on the generators the benchmark runs on (pcengine_b200/synth.py): the LiDAR-shaped scan's single
layers, the indoor-room sweep in both dataflows, the tiled scene with 3x3x3 and 5x5x5 kernels, and the
full-width network on one LiDAR scan.  Kernel maps bit-exact, features rel-L2 <= 1e-3 (fp16, fp32
accumulate), whole network <= 5e-3, against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import conv_oracle as co
from oracle import kmap_oracle as ko
from oracle import minkunet_oracle as mo

pytestmark = pytest.mark.gpu
TOL_FP16 = 1e-3
_CACHE = {}


def _lidar():
    from pcengine_b200 import synth
    if "lidar" not in _CACHE:
        coords = synth.with_batch(synth.lidar_scan(2000))
        cmax = coords[:, 1:].max(0).tolist()
        _CACHE["lidar"] = dict(
            coords=coords, cmax=cmax,
            subm=ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True),
            down=ko.build_d2(coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], cmax, False))
    return _CACHE["lidar"]


def _maps_equal(km, d2):
    assert np.array_equal(km.out_coords.cpu().numpy(), d2["out_coords"])
    assert np.array_equal(km.map.cpu().numpy(), d2["map"].reshape(-1))
    assert np.array_equal(km.knnz.cpu().numpy(), d2["knnz"])
    assert np.array_equal(km.kpos.cpu().numpy(), d2["kpos"]) and np.array_equal(km.qkpos.cpu().numpy(), d2["qkpos"])


def test_lidar_scan_kernel_maps_are_bit_exact():
    import pcengine_b200 as pce
    L = _lidar()
    dev_coords = torch.from_numpy(L["coords"]).cuda()
    km = pce.KernelMap(dev_coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], L["cmax"], True)
    _maps_equal(km, L["subm"])
    imap, omap = km.pairs()
    assert np.array_equal(imap.cpu().numpy(), L["subm"]["imap"]) and np.array_equal(omap.cpu().numpy(), L["subm"]["omap"])
    nb = ko.neighbour_csr(L["subm"])
    csr = km.csr()
    assert np.array_equal(csr.rowptr.cpu().numpy(), nb["rowptr"])
    assert np.array_equal(csr.nbr.cpu().numpy()[: int(nb["rowptr"][-1])], nb["nbr"])
    assert np.array_equal(csr.mask.cpu().numpy().view(np.uint32)[: len(nb["mask"])], nb["mask"])
    kd = pce.KernelMap(dev_coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], L["down"]["cmax_out"], False)
    _maps_equal(kd, L["down"])
    d1 = ko.build_d1(L["down"])
    imap_c, icsr, omap_c, ocsr = kd.d1()
    assert np.array_equal(icsr.cpu().numpy(), d1["icsr"]) and np.array_equal(imap_c.cpu().numpy(), d1["imap"])
    assert np.array_equal(ocsr.cpu().numpy(), d1["ocsr"]) and np.array_equal(omap_c.cpu().numpy(), d1["omap"])


@pytest.mark.parametrize("kind,cin,cout", [("subm", 32, 32), ("subm", 64, 64), ("subm", 128, 128), ("down", 32, 64),
                                           ("up", 64, 32)])
def test_lidar_scan_single_layers(kind, cin, cout):
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    L = _lidar()
    d2 = L["subm"] if kind == "subm" else L["down"]
    kv = d2["kv"]
    n_src = d2["n_out"] if kind == "up" else d2["n_in"]
    g = torch.Generator().manual_seed(2000 + cin)
    feats = torch.randn(n_src, cin, generator=g).half()
    w = (torch.randn(kv, cin, cout, generator=g) / (kv * cin) ** 0.5).half()
    dev_coords = torch.from_numpy(L["coords"]).cuda()
    if kind == "subm":
        km = pce.KernelMap(dev_coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], L["cmax"], True)
    else:
        km = pce.KernelMap(dev_coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], d2["cmax_out"], False)
    want = co.conv_forward(feats, w, d2, transposed=(kind == "up"))
    out = PF.conv_forward(feats.cuda(), w.cuda(), km.csr(transposed=(kind == "up")))
    assert co.rel_l2(out.float().cpu(), want) <= TOL_FP16
    out_d1 = PF.conv_forward_d1(feats.cuda(), w.cuda(), km, transposed=(kind == "up"))
    assert co.rel_l2(out_d1.float().cpu(), want) <= TOL_FP16
    assert PF.device_status() == 0


@pytest.mark.parametrize("c", [16, 32, 64, 96, 128, 256])
def test_indoor_room_sweep_both_dataflows(c):
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    from pcengine_b200 import synth
    if "room" not in _CACHE:
        xyz, _ = synth.indoor_room(3001, 40000)
        coords = synth.with_batch(xyz)
        cmax = coords[:, 1:].max(0).tolist()
        _CACHE["room"] = (coords, cmax, ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True))
    coords, cmax, d2 = _CACHE["room"]
    g = torch.Generator().manual_seed(3000 + c)
    feats = torch.randn(len(coords), c, generator=g).half()
    w = (torch.randn(27, c, c, generator=g) / (27 * c) ** 0.5).half()
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
    _maps_equal(km, d2)
    want = co.conv_forward(feats, w, d2)
    assert co.rel_l2(PF.conv_forward(feats.cuda(), w.cuda(), km.csr()).float().cpu(), want) <= TOL_FP16
    assert co.rel_l2(PF.conv_forward_d1(feats.cuda(), w.cuda(), km).float().cpu(), want) <= TOL_FP16
    assert PF.device_status() == 0


@pytest.mark.parametrize("ks", [3, 5])
def test_tiled_scene_two_rooms(ks):
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    from pcengine_b200 import synth
    coords = synth.with_batch(synth.tiled_scene(2, 1, voxels_per_room=30000))
    cmax = coords[:, 1:].max(0).tolist()
    d2 = ko.build_d2(coords, (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
    _maps_equal(km, d2)
    g = torch.Generator().manual_seed(5000 + ks)
    feats = torch.randn(len(coords), 64, generator=g).half()
    w = (torch.randn(ks ** 3, 64, 64, generator=g) / (ks ** 3 * 64) ** 0.5).half()
    out = PF.conv_forward(feats.cuda(), w.cuda(), km.csr())
    assert co.rel_l2(out.float().cpu(), co.conv_forward(feats, w, d2)) <= TOL_FP16
    assert PF.device_status() == 0


def test_full_width_network_on_one_lidar_scan():
    """MinkUNet(cr=1.0), fp16, on the scan of seed 2000: nine kernel maps bit-exact, logits <= 5e-3."""
    import pcengine_b200 as pce
    L = _lidar()
    coords = L["coords"]
    g = torch.Generator().manual_seed(4001)
    feats = torch.randn(len(coords), 4, generator=g).half()
    torch.manual_seed(4001)
    model = pce.MinkUNet(4, 19, cr=1.0)
    pce.randomize_batchnorm(model, 4001)
    model = model.half().eval()
    want, maps = mo.forward(model.state_dict(), coords, feats, return_maps=True)
    model = model.cuda()
    x = pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], L["cmax"],
                     init_tag=pce.MinkUNet.tags())
    with torch.no_grad():
        y = model(x)
    assert len(y.kmaps) == 9 == len(maps)
    ones = ko.encode3((1, 1, 1))
    for (ks_code, tstride, stride), km in y.kmaps.items():
        level = int(round(np.log2(ko.decode3(tstride)[0])))
        d2 = maps[("subm" if stride == ones else "down", level)]
        as_np = lambda a: (a.tensor() if hasattr(a, "tensor") else a).cpu().numpy()
        assert np.array_equal(as_np(km.map), d2["map"].reshape(-1)), (level, stride)
        assert np.array_equal(as_np(km.kpos), d2["kpos"]) and np.array_equal(as_np(km.qkpos), d2["qkpos"])
        assert np.array_equal(as_np(km.out_coords), d2["out_coords"])
    assert co.rel_l2(y.feats.float().cpu(), want) <= 5e-3
