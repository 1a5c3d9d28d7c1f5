"""Committed golden fixtures: the oracle must still reproduce them (CPU), and the CUDA path must match
them bit for bit in every map form and within tolerance in the features (GPU)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import conv_oracle as co
from oracle import kmap_oracle as ko
from tests.helpers import cmax_of

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FILES = sorted(f for f in glob.glob(os.path.join(HERE, "*.npz")) if not os.path.basename(f).startswith("ref_"))  # ref_*: tests/test_ref_golden.py


def _geom(g):
    return tuple(int(v) for v in g["ks"]), tuple(int(v) for v in g["stride"]), tuple(int(v) for v in g["pad"]), bool(g["subm"])


def test_fixtures_exist():
    assert len(FILES) >= 5


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(f)[:-4] for f in FILES])
def test_oracle_reproduces_golden(path):
    g = np.load(path)
    ks, stride, pad, subm = _geom(g)
    coords = g["coords"]
    d2 = ko.build_d2(coords, ks, stride, pad, [0, 0, 0], cmax_of(coords), subm)
    for key in ("out_coords", "map", "knnz", "kpos", "qkpos", "imap", "omap"):
        assert np.array_equal(d2[key], g[key]), key
    d1 = ko.build_d1(d2)
    assert np.array_equal(d1["icsr"], g["icsr"]) and np.array_equal(d1["imap"], g["imap_coded"])
    assert np.array_equal(d1["ocsr"], g["ocsr"]) and np.array_equal(d1["omap"], g["omap_coded"])
    nb = ko.neighbour_csr(d2)
    assert np.array_equal(nb["mask"], g["mask"]) and np.array_equal(nb["rowptr"], g["rowptr"])
    assert np.array_equal(nb["nbr"], g["nbr"])
    out = co.conv_forward(torch.from_numpy(g["feats"]), torch.from_numpy(g["weights"]), d2)
    assert co.rel_l2(out, torch.from_numpy(g["out"])) <= 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(f)[:-4] for f in FILES])
def test_cuda_path_matches_golden(path):
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    g = np.load(path)
    ks, stride, pad, subm = _geom(g)
    coords = g["coords"]
    cmax = cmax_of(coords)
    cmax_out = cmax if subm else [(cmax[i] + 2 * pad[i] - (ks[i] - 1)) // stride[i] for i in range(3)]
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), ks, stride, pad, [0, 0, 0], cmax_out, subm)
    assert np.array_equal(km.out_coords.cpu().numpy(), g["out_coords"])
    assert np.array_equal(km.map.cpu().numpy(), g["map"])
    assert np.array_equal(km.knnz.cpu().numpy(), g["knnz"])
    assert np.array_equal(km.kpos.cpu().numpy(), g["kpos"]) and np.array_equal(km.qkpos.cpu().numpy(), g["qkpos"])
    imap, omap = km.pairs()
    assert np.array_equal(imap.cpu().numpy(), g["imap"]) and np.array_equal(omap.cpu().numpy(), g["omap"])
    imap_c, icsr, omap_c, ocsr = km.d1()
    assert np.array_equal(icsr.cpu().numpy(), g["icsr"]) and np.array_equal(imap_c.cpu().numpy(), g["imap_coded"])
    assert np.array_equal(ocsr.cpu().numpy(), g["ocsr"]) and np.array_equal(omap_c.cpu().numpy(), g["omap_coded"])
    for tr, sfx in ((False, ""), (True, "_t")):
        csr = km.csr(transposed=tr)
        n = len(g["rowptr" + sfx]) - 1
        assert np.array_equal(csr.rowptr.cpu().numpy(), g["rowptr" + sfx])
        assert np.array_equal(csr.mask.cpu().numpy().view(np.uint32)[:n], g["mask" + sfx])
        assert np.array_equal(csr.nbr.cpu().numpy()[: int(g["rowptr" + sfx][-1])], g["nbr" + sfx])
    feats = torch.from_numpy(g["feats"]).cuda()
    for choice in ("auto", "simt"):
        out = PF.conv_forward(feats, torch.from_numpy(g["weights"]).cuda(), km.csr(), None, choice)
        assert co.rel_l2(out.float().cpu(), torch.from_numpy(g["out"])) <= 1e-3
        back = PF.conv_forward(torch.from_numpy(g["out"]).half().cuda(), torch.from_numpy(g["back_weights"]).cuda(),
                               km.csr(transposed=True), None, choice)
        assert co.rel_l2(back.float().cpu(), torch.from_numpy(g["back"])) <= 1e-3
    assert PF.device_status() == 0
