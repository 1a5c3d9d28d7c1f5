"""The five ``backend`` entry points called exactly as the reference's Python layer calls
them (script/spconv.py:345-376 for D2, :390-434 for D1, :240-253 / :146-161 for the
forwards), following the flow of the reference's check_fwd.py with the CPU oracle in the
place of its third-party comparator (GPU)."""
import numpy as np
import pytest
import torch

from oracle import conv_oracle as co
from oracle import kmap_oracle as ko
from tests.helpers import cmax_of, random_cloud, surface_cloud

pytestmark = pytest.mark.gpu


def _enc(v):
    return 94273 * v[0] + 311 * v[1] + v[2]


def _coordinate_hash(c):
    return c[:, 1].long() * (2 ** 20) + c[:, 2].long() * (2 ** 10) + c[:, 3].long()


@pytest.mark.parametrize("dtype,cin,cout", [(torch.float32, 16, 16), (torch.float16, 64, 64), (torch.float16, 32, 64)])
@pytest.mark.parametrize("ks,stride", [(3, 1), (3, 2), (2, 2)])
def test_fetch_on_demand_flow(dtype, cin, cout, ks, stride):
    from pcengine_b200.backend import conv_fwd_d2_cuda, mapping_d2_cuda
    dev = torch.device("cuda:0")
    coords = surface_cloud(21, 60, batch=2)
    n, kv = len(coords), ks ** 3
    torch.manual_seed(3)
    feats = torch.rand(n, cin).to(dtype)
    kernel = torch.rand(kv, cin, cout).to(dtype)
    subm = stride == 1
    cmax = cmax_of(coords)
    cmax_out = cmax if subm else [(cmax[i] - (ks - 1)) // stride for i in range(3)]
    dcoords = torch.from_numpy(coords).to(dev)
    imap = -torch.ones(kv * n, dtype=torch.int, device=dev)
    knnz = torch.zeros(kv, dtype=torch.int, device=dev)
    kpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    qkpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    out_coords = mapping_d2_cuda(dcoords, 2, _enc([ks] * 3), kv, cin, cout, _enc([stride] * 3), _enc([1, 1, 1]),
                                 _enc([0, 0, 0]), 0, 0, 0, cmax_out[0], cmax_out[1], cmax_out[2], imap, knnz, kpos,
                                 qkpos, subm)
    if subm:
        assert out_coords is dcoords
    nonzero_idx = torch.nonzero(imap != -1)
    omap = imap[nonzero_idx]
    imap_p = (nonzero_idx % n).int()
    qsum = qkpos[-1].cpu().int()
    d2 = ko.build_d2(coords, (ks,) * 3, (stride,) * 3, (0, 0, 0), [0, 0, 0], cmax, subm)
    assert np.array_equal(imap.cpu().numpy(), d2["map"]) and int(qsum) == d2["qsum"]
    assert np.array_equal(knnz.cpu().numpy(), d2["knnz"]) and np.array_equal(kpos.cpu().numpy(), d2["kpos"])
    n_out = out_coords.size(0)
    out = torch.zeros((n_out, cout), dtype=dtype, device=dev)
    conv_fwd_d2_cuda(feats.to(dev), kernel.to(dev), _enc([ks] * 3), qsum, out, kpos, qkpos, imap_p, omap, subm, True)
    ref = co.conv_forward(feats, kernel, d2)
    # compare after sorting both sides by the coordinate hash, as check_fwd.py does
    i1 = torch.sort(_coordinate_hash(out_coords.cpu()) + out_coords.cpu()[:, 0].long() * 2 ** 40).indices
    oc = torch.from_numpy(d2["out_coords"])
    i2 = torch.sort(_coordinate_hash(oc) + oc[:, 0].long() * 2 ** 40).indices
    assert torch.equal(out_coords.cpu()[i1], oc[i2])
    a, b = out.float().cpu()[i1], ref[i2]
    rtol, atol = (1e-2, 1e-4) if dtype == torch.half else (1e-3, 1e-6)
    assert torch.allclose(a, b, rtol=rtol, atol=atol * max(1.0, float(b.abs().max())))
    assert co.rel_l2(a, b) <= (1e-3 if dtype == torch.half else 1e-5)
    # transposed use: maps swapped (script/spconv.py:236-244)
    if not subm:
        back = torch.zeros((n, cin), dtype=dtype, device=dev)
        kt = torch.rand(kv, cout, cin).to(dtype)
        conv_fwd_d2_cuda(out, kt.to(dev), _enc([ks] * 3), qsum, back, kpos, qkpos, omap, imap_p, False, True)
        refb = co.conv_forward(out.cpu(), kt, d2, transposed=True)
        assert co.rel_l2(back.float().cpu(), refb) <= (1e-3 if dtype == torch.half else 1e-5)


@pytest.mark.parametrize("dtype,cin,cout", [(torch.float32, 16, 16), (torch.float16, 64, 32)])
@pytest.mark.parametrize("ks,stride", [(3, 1), (3, 2), (2, 2)])
def test_gather_mm_scatter_flow(dtype, cin, cout, ks, stride):
    from pcengine_b200.backend import conv_fwd_d1_cuda, mapping_d1_cuda
    dev = torch.device("cuda:0")
    coords = random_cloud(13, 28, 5000, batch=2)
    n, kv = len(coords), ks ** 3
    torch.manual_seed(4)
    feats = torch.rand(n, cin).to(dtype)
    kernel = (torch.rand(kv, cin, cout) / cin).to(dtype)
    subm = stride == 1
    cmax = cmax_of(coords)
    cmax_out = cmax if subm else [(cmax[i] - (ks - 1)) // stride for i in range(3)]
    dcoords = torch.from_numpy(coords).to(dev)
    imap = -torch.ones(n * kv, dtype=torch.int, device=dev)
    omap = -torch.ones(n * kv * 8, dtype=torch.int, device=dev)
    knnz = torch.zeros(kv, dtype=torch.int, device=dev)
    kpos = torch.zeros(kv, dtype=torch.int, device=dev)  # the reference allocates kv, not kv+1
    qkpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    icsr = torch.zeros(n + 2, dtype=torch.int, device=dev)
    ocsr = torch.zeros((n + 2) * 8, dtype=torch.int, device=dev)
    out_coords = mapping_d1_cuda(dcoords, _enc([ks] * 3), kv, cin, cout, _enc([stride] * 3), _enc([1, 1, 1]),
                                 _enc([0, 0, 0]), 0, 0, 0, cmax_out[0], cmax_out[1], cmax_out[2], imap, omap, icsr,
                                 ocsr, knnz, kpos, qkpos, subm)
    d2 = ko.build_d2(coords, (ks,) * 3, (stride,) * 3, (0, 0, 0), [0, 0, 0], cmax, subm)
    d1 = ko.build_d1(d2)
    p, n_out = len(d2["imap"]), d2["n_out"]
    assert np.array_equal(out_coords.cpu().numpy(), d2["out_coords"])
    assert np.array_equal(icsr.cpu().numpy()[: n + 1], d1["icsr"])
    assert np.array_equal(ocsr.cpu().numpy()[: n_out + 1], d1["ocsr"])
    assert np.array_equal(imap.cpu().numpy()[:p], d1["imap"]) and np.array_equal(omap.cpu().numpy()[:p], d1["omap"])
    assert np.array_equal(kpos.cpu().numpy(), d2["kpos"][:kv]) and np.array_equal(qkpos.cpu().numpy(), d2["qkpos"])
    qsum = qkpos[-1].cpu().int()
    buffer = torch.zeros((int(qsum), cin + cout), dtype=dtype, device=dev)
    out = torch.zeros((n_out, cout), dtype=dtype, device=dev)
    conv_fwd_d1_cuda(feats.to(dev), kernel.to(dev), _enc([ks] * 3), qsum, out, kpos, qkpos, imap, omap, icsr, ocsr,
                     buffer, subm, 1)
    ref = co.conv_forward(feats, kernel, d2)
    assert co.rel_l2(out.float().cpu(), ref) <= (1e-3 if dtype == torch.half else 1e-5)


def test_backward_entry_point_raises():
    from pcengine_b200.backend import conv_bwd_d1_cuda
    with pytest.raises(NotImplementedError):
        conv_bwd_d1_cuda()
