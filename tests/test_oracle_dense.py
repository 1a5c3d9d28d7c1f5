"""Pins the CPU oracle against dense torch conv3d on small grids (CPU only)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import conv_oracle as co
from oracle import kmap_oracle as ko


def _cloud(rng, d, n, batch=1):
    out = []
    for b in range(batch):
        lin = rng.choice(d ** 3, n, replace=False)
        xyz = np.stack([lin // (d * d), (lin // d) % d, lin % d], 1)
        out.append(np.concatenate([np.full((n, 1), b), xyz], 1))
    return np.concatenate(out).astype(np.int32)


def _dense(coords, feats, shape, batch):
    g = torch.zeros((batch, feats.shape[1]) + tuple(shape), dtype=feats.dtype)
    c = torch.from_numpy(coords.astype(np.int64))
    g[c[:, 0], :, c[:, 1], c[:, 2], c[:, 3]] = feats
    return g


def _dense_weight(w, ks):
    return w.reshape(*ks, w.shape[1], w.shape[2]).permute(4, 3, 0, 1, 2).contiguous()


@pytest.mark.parametrize("ks", [(3, 3, 3), (5, 5, 5), (3, 1, 5)])
@pytest.mark.parametrize("batch", [1, 2])
def test_submanifold_equals_dense(ks, batch):
    rng = np.random.default_rng(7)
    torch.manual_seed(7)
    d, n, ci, cout = 11, 260, 5, 7
    coords = _cloud(rng, d, n, batch)
    feats = torch.randn(len(coords), ci, dtype=torch.float64)
    kv = ks[0] * ks[1] * ks[2]
    w = torch.randn(kv, ci, cout, dtype=torch.float64)
    cmax = coords[:, 1:].max(0).tolist()
    d2 = ko.build_d2(coords, ks, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
    out = co.conv_forward(feats, w, d2).double()
    # fp32 oracle arithmetic: compare to an fp32 dense conv
    ref = F.conv3d(_dense(coords, feats.float(), (d, d, d), batch), _dense_weight(w.float(), ks),
                   padding=tuple((k - 1) // 2 for k in ks))
    c = torch.from_numpy(coords.astype(np.int64))
    refs = ref[c[:, 0], :, c[:, 1], c[:, 2], c[:, 3]].double()
    assert co.rel_l2(out, refs) < 1e-6


@pytest.mark.parametrize("ks,stride,pad", [((3, 3, 3), (2, 2, 2), (0, 0, 0)), ((3, 3, 3), (2, 2, 2), (1, 1, 1)),
                                           ((2, 2, 2), (2, 2, 2), (0, 0, 0)), ((2, 2, 2), (1, 2, 2), (0, 0, 0)),
                                           ((3, 3, 3), (3, 3, 3), (0, 0, 0))])
def test_strided_equals_dense(ks, stride, pad):
    rng = np.random.default_rng(11)
    torch.manual_seed(11)
    d, n, ci, cout, batch = 12, 300, 4, 6, 2
    coords = _cloud(rng, d, n, batch)
    feats = torch.randn(len(coords), ci)
    kv = ks[0] * ks[1] * ks[2]
    w = torch.randn(kv, ci, cout)
    cmax = [d - 1] * 3
    d2 = ko.build_d2(coords, ks, stride, pad, [0, 0, 0], cmax, False)
    out = co.conv_forward(feats, w, d2)
    ref = F.conv3d(_dense(coords, feats, (d, d, d), batch), _dense_weight(w, ks), stride=stride, padding=pad)
    oc = torch.from_numpy(d2["out_coords"].astype(np.int64))
    assert (oc[:, 1] < ref.shape[2]).all() and (oc[:, 2] < ref.shape[3]).all() and (oc[:, 3] < ref.shape[4]).all()
    refs = ref[oc[:, 0], :, oc[:, 1], oc[:, 2], oc[:, 3]]
    assert co.rel_l2(out, refs) < 1e-6
    # every non-zero dense output location is an output voxel
    nz = (ref.abs().sum(1) > 0).sum().item()
    assert nz <= len(oc)
    # sorted ascending (b,x,y,z), unique
    code = ((oc[:, 0] * 4096 + oc[:, 1]) * 4096 + oc[:, 2]) * 4096 + oc[:, 3]
    assert (code[1:] > code[:-1]).all()


def test_transposed_is_adjoint_of_strided():
    """<conv_T(y), x> == <y, conv(x)> with the same weights (maps swapped)."""
    rng = np.random.default_rng(3)
    torch.manual_seed(3)
    coords = _cloud(rng, 10, 200, 1)
    ks, st = (2, 2, 2), (2, 2, 2)
    d2 = ko.build_d2(coords, ks, st, (0, 0, 0), [0, 0, 0], [9, 9, 9], False)
    ci, cout = 3, 5
    w = torch.randn(8, ci, cout)
    x = torch.randn(len(coords), ci)
    y = torch.randn(d2["n_out"], cout)
    fwd = co.conv_forward(x, w, d2)
    bwd = co.conv_forward(y, w.transpose(1, 2).contiguous(), d2, transposed=True)
    assert abs(float((fwd * y).sum() - (bwd * x).sum())) < 1e-3
    assert bwd.shape == (len(coords), ci)


def test_scans_and_d1_forms():
    rng = np.random.default_rng(5)
    coords = _cloud(rng, 8, 150, 1)
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], [7, 7, 7], True)
    assert d2["knnz"][13] == 0 and d2["kpos"][-1] == len(d2["imap"])
    assert d2["qsum"] % 128 == 0 and d2["qsum"] >= d2["kpos"][-1]
    # symmetric offsets have equal counts in a submanifold map
    assert (d2["knnz"] == d2["knnz"][::-1]).all()
    d1 = ko.build_d1(d2)
    assert d1["icsr"][-1] == len(d2["imap"]) == d1["ocsr"][-1]
    kp = d1["omap"] // ko.D1_CODE
    for r in range(d2["n_out"]):
        seg = kp[d1["ocsr"][r]:d1["ocsr"][r + 1]]
        assert (np.diff(seg) > 0).all()
    # decoding a code gives back the pair
    pos = d1["imap"] % ko.D1_CODE + d2["kpos"][d1["imap"] // ko.D1_CODE]
    rows = np.repeat(np.arange(d2["n_in"]), np.diff(d1["icsr"]))
    assert (d2["imap"][pos] == rows).all()
    nb = ko.neighbour_csr(d2)
    assert nb["rowptr"][-1] == len(d2["imap"]) + d2["n_in"]
    assert (nb["mask"][:, 0] >> 13 & 1).all()
