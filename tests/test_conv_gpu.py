"""Feature parity of the CUDA convolutions against the CPU oracle (GPU).
Tolerances: rel-L2 <= 1e-5 for fp32, <= 1e-3 for fp16 (fp32 accumulate)."""
import numpy as np
import pytest
import torch

from oracle import conv_oracle as co
from oracle import kmap_oracle as ko
from tests.helpers import cmax_of, random_cloud, surface_cloud

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.float16: 1e-3}


def _tensor(pce, coords, feats, tags=("D2", "D2", "D2", "end")):
    dev = torch.device("cuda:0")
    return pce.spTensor(feats.to(dev), torch.from_numpy(coords).to(dev), None, [0, 0, 0], cmax_of(coords),
                        init_tag=list(tags))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("cin,cout", [(16, 16), (4, 32), (32, 32), (64, 64), (32, 64), (96, 96), (128, 128), (24, 19),
                                      (3, 5), (160, 48), (224, 256)])
@pytest.mark.parametrize("kernel_choice", ["auto", "simt"])
def test_submanifold_features(dtype, cin, cout, kernel_choice):
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(3, 72, batch=2)
    torch.manual_seed(1)
    feats = torch.randn(len(coords), cin).to(dtype)
    w = (torch.randn(27, cin, cout) / (27 * cin) ** 0.5).to(dtype)
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    out = PF.conv_forward(feats.cuda(), w.cuda(), km.csr(), None, kernel_choice)
    ref = co.conv_forward(feats, w, d2)
    assert co.rel_l2(out.float().cpu(), ref) <= TOL[dtype]
    # run to run the result is bit-identical (no atomics anywhere)
    out2 = PF.conv_forward(feats.cuda(), w.cuda(), km.csr(), None, kernel_choice)
    assert torch.equal(out, out2)


def test_config1_fp32_c16():
    """The fp32 benchmark case: 20,000 voxels in 64^3, C 16->16, weights N(0, 1/(27*16))."""
    import pcengine_b200 as pce
    from pcengine_b200 import synth
    coords = synth.with_batch(synth.uniform_grid(20000, 64, 1001))
    g = torch.Generator().manual_seed(1001)
    feats = torch.randn(20000, 16, generator=g)
    w = torch.randn(27, 16, 16, generator=g) / (27 * 16) ** 0.5
    x = _tensor(pce, coords, feats)
    conv = pce.conv3d(16, 16, 3, 1).cuda()
    conv.kernel.data.copy_(w)
    y = conv(x)
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    km = x.kmaps[(conv.kernel_size_code, x.stride, conv.stride_code)]
    assert np.array_equal(km.map.cpu().numpy(), d2["map"])
    assert co.rel_l2(y.feats.cpu(), co.conv_forward(feats, w, d2)) <= 1e-5
    assert y.coords.data_ptr() == x.coords.data_ptr()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("ks,stride,pad,cin,cout", [(2, 2, 0, 32, 64), (3, 2, 1, 16, 32), (3, 2, 0, 8, 8)])
def test_strided_then_transposed(dtype, ks, stride, pad, cin, cout):
    import pcengine_b200 as pce
    coords = random_cloud(9, 40, 9000, batch=2)
    torch.manual_seed(2)
    feats = torch.randn(len(coords), cin).to(dtype)
    x = _tensor(pce, coords, feats)
    down = pce.conv3d(cin, cout, ks, stride, pad, bias=True).cuda().to(dtype)
    up = pce.conv3d(cout, cin, ks, stride, pad, transposed=True).cuda().to(dtype)
    z = down(x)
    u = up(z)
    d2 = ko.build_d2(coords, (ks,) * 3, (stride,) * 3, (pad,) * 3, [0, 0, 0], cmax_of(coords), False)
    assert np.array_equal(z.coords.cpu().numpy(), d2["out_coords"])
    assert z.stride == pce.conv_info_encoder([stride] * 3) and u.stride == x.stride
    assert list(z.coords_max) == list(d2["cmax_out"])
    refz = co.conv_forward(feats, down.kernel.detach().cpu(), d2, bias=down.bias.detach().cpu())
    assert co.rel_l2(z.feats.float().cpu(), refz) <= TOL[dtype]
    refu = co.conv_forward(z.feats.cpu(), up.kernel.detach().cpu(), d2, transposed=True)
    assert co.rel_l2(u.feats.float().cpu(), refu) <= TOL[dtype]
    assert u.coords.data_ptr() == x.coords.data_ptr() and u.feats.shape == (len(coords), cin)


def test_kmap_cache_and_tags():
    import pcengine_b200 as pce
    coords = random_cloud(4, 20, 1500)
    feats = torch.randn(len(coords), 8)
    x = _tensor(pce, coords, feats, tags=("D2", "end"))
    c1 = pce.conv3d(8, 8, 3).cuda()
    c2 = pce.conv3d(8, 8, 3).cuda()
    y = c1(x)
    assert y.init_tag == ["end"] and len(y.kmaps) == 1
    z = c2(y)  # same key: cached map, no tag consumed
    assert len(z.kmaps) == 1 and z.kmaps is x.kmaps
    with pytest.raises(NotImplementedError):
        pce.conv3d(8, 8, 5).cuda()(z)  # new map needed but the tag list is exhausted
    with pytest.raises(RuntimeError):
        pce.conv3d(8, 8, 2, 2, transposed=True).cuda()(z)  # no matching strided map
    with pytest.raises(ValueError):
        pce.conv3d(4, 8, 3).cuda()(z)  # channel mismatch


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_fused_epilogue_bn_relu_residual_and_modules(dtype):
    import pcengine_b200 as pce
    coords = surface_cloud(8, 48)
    torch.manual_seed(5)
    c = 32
    feats = torch.randn(len(coords), c).to(dtype)
    x = _tensor(pce, coords, feats)
    conv = pce.conv3d(c, c, 3, bias=True).cuda().to(dtype)
    bn = pce.BatchNorm(c).cuda()
    bn.running_mean.uniform_(-0.5, 0.5)
    bn.running_var.uniform_(0.5, 2.0)
    bn.weight.data.uniform_(0.5, 1.5)
    bn.bias.data.uniform_(-0.5, 0.5)
    bn.eval()
    relu = pce.ReLU()
    leaky = pce.LeakyReLU(0.1)
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    raw = co.conv_forward(feats, conv.kernel.detach().cpu(), d2, bias=conv.bias.detach().cpu())
    bnref = co.batchnorm_eval(raw, bn.weight.cpu(), bn.bias.cpu(), bn.running_mean.cpu(), bn.running_var.cpu(), bn.eps)
    # unfused modules
    y = relu(bn(conv(x)))
    assert co.rel_l2(y.feats.float().cpu(), torch.relu(bnref)) <= TOL[dtype] * 2
    y2 = leaky(bn(conv(x)))
    assert co.rel_l2(y2.feats.float().cpu(), co.activation(bnref, "leaky", 0.1)) <= TOL[dtype] * 2
    # fused into the convolution's store
    scale, shift = pce.bn_scale_shift(bn)
    res = torch.randn(len(coords), c).to(dtype)
    ep = pce.FusedEpilogue(scale=scale, shift=shift, residual=res.cuda(), act="relu")
    yf = conv(x, epilogue=ep)
    assert co.rel_l2(yf.feats.float().cpu(), torch.relu(bnref + res.float())) <= TOL[dtype]
    # cat / add keep coordinates and maps
    s = pce.cat([y, y2])
    assert s.feats.shape[1] == 2 * c and s.kmaps is x.kmaps
    a = y + y2
    assert torch.allclose(a.feats, y.feats + y2.feats)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_pointwise_conv(dtype):
    import pcengine_b200 as pce
    coords = random_cloud(6, 16, 1000)
    feats = torch.randn(len(coords), 96).to(dtype)
    x = _tensor(pce, coords, feats)
    head = pce.conv3d(96, 19, 1, bias=True).cuda().to(dtype)
    y = head(x)
    ref = co.pointwise_conv(feats, head.kernel.detach().cpu(), head.bias.detach().cpu())
    assert co.rel_l2(y.feats.float().cpu(), ref) <= TOL[dtype]
    assert len(y.kmaps) == 0


def test_5x5x5_submanifold_fp16():
    import pcengine_b200 as pce
    coords = surface_cloud(12, 40)
    feats = torch.randn(len(coords), 64).half()
    x = _tensor(pce, coords, feats)
    conv = pce.conv3d(64, 64, 5).cuda().half()
    y = conv(x)
    d2 = ko.build_d2(coords, (5, 5, 5), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    assert co.rel_l2(y.feats.float().cpu(), co.conv_forward(feats, conv.kernel.detach().cpu(), d2)) <= 1e-3


def test_weight_repacking_follows_the_tensor():
    """Fresh weight tensors that reuse a freed allocation, and in-place updates, must never meet
    a stale tensor-core layout."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(2, 40)
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    x = torch.randn(len(coords), 32).half()
    xd = x.cuda()
    for scale in (1.0, 0.05, 3.0):
        w = (torch.rand(27, 32, 32) * scale).half()
        wd = w.cuda()
        y = PF.conv_forward(xd, wd, km.csr())
        assert co.rel_l2(y.float().cpu(), co.conv_forward(x, w, d2)) <= 1e-3
        wd.mul_(0.5)  # in-place update bumps the version counter
        y = PF.conv_forward(xd, wd, km.csr())
        assert co.rel_l2(y.float().cpu(), co.conv_forward(x, w * 0.5, d2)) <= 1e-3
        del wd, y
    assert PF.device_status() == 0


def test_row_order_is_only_scheduling():
    """Tiles formed in the sorted order give bit-identical features to natural order, and the order is
    a permutation grouped by bitmask."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(9, 80, batch=2)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    csr = km.csr()
    order = csr.order().cpu().numpy()
    assert np.array_equal(np.sort(order), np.arange(km.n_out))
    keys = csr.mask.cpu().numpy().view(np.uint32)[:, 0][order]
    # rows with the same bitmask are contiguous in the order (the sort key is a bijection of the mask)
    assert np.count_nonzero(np.diff(keys.astype(np.int64))) == len(np.unique(keys)) - 1
    x = torch.randn(len(coords), 64).half().cuda()
    w = (torch.randn(27, 64, 96) / 40).half().cuda()
    try:
        PF.SORT_ROWS = True
        a = PF.conv_forward(x, w, csr)
        PF.SORT_ROWS = False
        b = PF.conv_forward(x, w, csr)
    finally:
        PF.SORT_ROWS = True
    assert torch.equal(a, b)
    assert PF.device_status() == 0


@pytest.mark.parametrize("cin,cout,ks", [(64, 64, 3), (96, 128, 3), (256, 256, 3), (32, 48, 5), (128, 32, 2)])
def test_tile_height_is_only_scheduling(cin, cout, ks):
    """256-row tiles (two accumulators per staged weight block) give the same features as 128-row
    tiles, bit for bit: every output row still sums its offsets in ascending order in fp32."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(11, 72, batch=2)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    csr = km.csr()
    g = torch.Generator().manual_seed(cin * 7 + cout)
    x = torch.randn(len(coords), cin, generator=g).half().cuda()
    w = (torch.randn(ks ** 3, cin, cout, generator=g) / 30).half().cuda()
    ep = PF.FusedEpilogue(scale=torch.rand(cout, generator=g).cuda() + 0.5, shift=torch.randn(cout, generator=g).cuda(),
                          act="relu")
    from pcengine_b200 import _lib
    outs = {}
    try:
        for rows in (128, 256, 512):
            if rows == 512 and (cout > 128 or cin < 64):
                continue  # four accumulators need <= 128 columns each; 512-row lists hold one offset per stage
            PF.TILE_ROWS = rows
            _lib.lib.pce_tune(4, 1)  # several accumulators per CTA, decoupled row / weight rings
            outs[("mt", rows)] = PF.conv_forward(x, w, csr, ep)
            _lib.lib.pce_tune(4, 0)  # the one-accumulator kernel (the default)
            if rows <= 256:
                outs[("single", rows)] = PF.conv_forward(x, w, csr, ep)
    finally:
        PF.TILE_ROWS = None
        _lib.lib.pce_tune(4, 0)
    assert (128 in [k[1] for k in csr._tiles]) and (256 in [k[1] for k in csr._tiles])
    a = b = outs[("mt", 128)]
    for key, o in outs.items():
        assert torch.equal(a, o), key
    d2 = ko.build_d2(coords, (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    want = co.conv_forward(x.float().cpu(), w.float().cpu(), d2)
    want = torch.relu(want * ep.scale.cpu() + ep.shift.cpu())
    assert co.rel_l2(b.float().cpu(), want) <= 1e-3  # fp16 features, fp32 accumulation
    assert PF.device_status() == 0


@pytest.mark.parametrize("cin,cout", [(4, 32), (24, 19), (3, 5)])
def test_ragged_channels_run_on_tensor_cores(cin, cout):
    """fp16 layers whose widths are not multiples of 16 are zero-padded onto the tensor-core kernel;
    the result has the unpadded shape, is contiguous and agrees with the CUDA-core kernel."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(5, 64, batch=2)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    g = torch.Generator().manual_seed(17)
    x = torch.randn(len(coords), cin, generator=g).half().cuda()
    w = (torch.randn(27, cin, cout, generator=g) / (27 * cin) ** 0.5).half().cuda()
    ep = PF.FusedEpilogue(scale=(torch.rand(cout, generator=g) + 0.5).cuda(), shift=torch.randn(cout, generator=g).cuda(),
                          act="leaky", slope=0.1)
    PF.PROFILE = []
    try:
        a = PF.conv_forward(x, w, km.csr(), ep)
        kernels = [r["kernel"] for r in PF.PROFILE]
    finally:
        PF.PROFILE = None
    assert kernels == ["conv_umma"]
    b = PF.conv_forward(x, w, km.csr(), ep, "simt")
    assert a.shape == (len(coords), cout) and a.is_contiguous()
    assert co.rel_l2(a.float().cpu(), b.float().cpu()) <= 1e-3
    # the padded weights are cached on the tensor and refreshed when it changes in place
    with torch.no_grad():
        w.mul_(2.0)
    c = PF.conv_forward(x, w, km.csr(), ep)
    d = PF.conv_forward(x, w, km.csr(), ep, "simt")
    assert co.rel_l2(c.float().cpu(), d.float().cpu()) <= 1e-3
    assert PF.device_status() == 0


@pytest.mark.parametrize("cin,cout,c2,ks,tile_rows", [(64, 64, 64, 3, 128), (96, 96, 128, 3, 128), (32, 32, 32, 3, 256),
                                                       (128, 256, 384, 3, 128), (48, 80, 16, 5, 128), (96, 96, 128, 3, 512),
                                                       (128, 128, 192, 3, 512), (256, 256, 256, 3, 256), (64, 32, 64, 3, None)])
def test_second_operand_joins_the_accumulator(cin, cout, c2, ks, tile_rows):
    """FusedEpilogue.extra_feats: out = act((conv(x) + x2 @ w2) * scale + shift), against the oracle's
    convolution plus a dense product, and bit-identical between the two tile heights' code paths and
    to itself run to run."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(21, 64, batch=2)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    csr = km.csr()
    g = torch.Generator().manual_seed(cin + 3 * cout + c2)
    n = len(coords)
    x = torch.randn(n, cin, generator=g).half()
    w = (torch.randn(ks ** 3, cin, cout, generator=g) / (ks ** 3 * cin) ** 0.5).half()
    x2 = torch.randn(n, c2, generator=g).half()
    w2 = (torch.randn(c2, cout, generator=g) / c2 ** 0.5).half()
    scale, shift = torch.rand(cout, generator=g) + 0.5, torch.randn(cout, generator=g)
    ep = PF.FusedEpilogue(scale=scale.cuda(), shift=shift.cuda(), act="relu", extra_feats=x2.cuda(), extra_weight=w2.cuda())
    plain = PF.FusedEpilogue(scale=scale.cuda(), shift=shift.cuda(), act="relu")
    from pcengine_b200 import _lib
    try:
        PF.TILE_ROWS = tile_rows
        a = PF.conv_forward(x.cuda(), w.cuda(), csr, ep)
        b = PF.conv_forward(x.cuda(), w.cuda(), csr, ep)
        c = PF.conv_forward(x.cuda(), w.cuda(), csr, plain)  # served by the lists that have the identity stage
        _lib.lib.pce_tune(4, 1)  # the kernel with several accumulators per CTA takes the second operand the same way
        a_mt = PF.conv_forward(x.cuda(), w.cuda(), csr, ep)
        c_mt = PF.conv_forward(x.cuda(), w.cuda(), csr, plain)
    finally:
        PF.TILE_ROWS = None
        _lib.lib.pce_tune(4, 0)
    assert torch.equal(a, b) and torch.equal(a, a_mt) and torch.equal(c, c_mt)
    d2 = ko.build_d2(coords, (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    want = torch.relu((co.conv_forward(x.float(), w.float(), d2) + x2.float() @ w2.float()) * scale + shift)
    assert co.rel_l2(a.float().cpu(), want) <= 1e-3  # fp16 operands, fp32 accumulation
    # the lists with the identity stage also served the launch without a second operand
    assert any(k[2] for k in csr._tiles) and not any(not k[2] for k in csr._tiles)
    assert co.rel_l2(c.float().cpu(), torch.relu(co.conv_forward(x.float(), w.float(), d2) * scale + shift)) <= 1e-3
    with pytest.raises(NotImplementedError):
        PF.conv_forward(x.cuda(), w.cuda(), csr, ep, "simt")
    with pytest.raises(NotImplementedError):
        PF.conv_forward(x.float().cuda(), w.float().cuda(), csr,
                        PF.FusedEpilogue(extra_feats=x2.float().cuda(), extra_weight=w2.float().cuda()))
    assert PF.device_status() == 0

@pytest.mark.gpu
def test_overlapped_launches_keep_the_stream_order():
    """Programmatic dependent launch (a convolution's set-up overlaps the previous kernel's tail): a chain
    of layers in which every launch reads what the launch before it wrote gives the same bits with the
    overlap on and off, run after run."""
    import pcengine_b200 as pce
    from pcengine_b200 import _lib
    from pcengine_b200 import functional as PF
    coords = surface_cloud(9, 96, batch=4)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    csr = km.csr()
    g = torch.Generator().manual_seed(99)
    widths = [32, 64, 96, 64, 128, 32, 16, 64]
    x0 = torch.randn(len(coords), widths[0], generator=g).half().cuda()
    ws = [(torch.randn(27, a, b, generator=g) / (27 * a) ** 0.5).half().cuda() for a, b in zip(widths[:-1], widths[1:])]

    def chain():
        x = x0
        for w in ws:
            x = PF.conv_forward(x, w, csr, PF.FusedEpilogue(act="relu"))
        return x
    try:
        _lib.lib.pce_tune(3, 0)
        want = chain()
        _lib.lib.pce_tune(3, 1)
        for _ in range(5):
            assert torch.equal(chain(), want)
    finally:
        _lib.lib.pce_tune(3, 1)
    assert PF.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("cin,cout,ks", [(64, 64, 3), (32, 96, 3), (16, 32, 3), (96, 96, 2), (128, 256, 3)])
def test_column_ranges_of_wider_matrices(cin, cout, ks):
    """Row pitches: the input read from, and the output written into, a column range of a wider
    row-major matrix give the bits of the dense call, and the columns beside the range stay untouched."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords = surface_cloud(33, 64, batch=2)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    csr = km.csr()
    g = torch.Generator().manual_seed(7 * cin + cout)
    n = len(coords)
    x = torch.randn(n, cin, generator=g).half().cuda()
    w = (torch.randn(ks ** 3, cin, cout, generator=g) / (ks ** 3 * cin) ** 0.5).half().cuda()
    ep = PF.FusedEpilogue(scale=(torch.rand(cout, generator=g) + 0.5).cuda(), shift=torch.randn(cout, generator=g).cuda(),
                          act="relu")
    want = PF.conv_forward(x, w, csr, ep)
    wide_in = torch.full((n, cin + 40), 7.0, dtype=torch.float16, device="cuda")
    wide_in[:, 8:8 + cin] = x
    wide_out = torch.full((n, cout + 24), -3.0, dtype=torch.float16, device="cuda")
    got = PF.conv_forward(wide_in[:, 8:8 + cin], w, csr, ep, out=wide_out[:, 16:16 + cout])
    assert got.data_ptr() == wide_out[:, 16:].data_ptr()  # written in place, no copy
    assert torch.equal(got, want)
    assert bool((wide_out[:, :16] == -3.0).all()) and bool((wide_out[:, 16 + cout:] == -3.0).all())
    # a range the kernel cannot address in place (odd column offset) goes through a copy, same values
    odd_out = torch.zeros((n, cout + 3), dtype=torch.float16, device="cuda")
    got = PF.conv_forward(wide_in[:, 8:8 + cin], w, csr, ep, out=odd_out[:, 3:])
    assert torch.equal(got, want) and torch.equal(odd_out[:, 3:], want)
    # the CUDA-core path takes the same arguments
    ref32 = PF.conv_forward(x.float(), w.float(), csr, ep, "simt")
    out32 = torch.zeros((n, cout + 8), dtype=torch.float32, device="cuda")
    PF.conv_forward(wide_in[:, 8:8 + cin].float(), w.float(), csr, ep, "simt", out=out32[:, 8:])
    assert torch.equal(out32[:, 8:], ref32)
    with pytest.raises(ValueError):
        PF.conv_forward(x, w, csr, ep, out=torch.empty((n, cout + 1), dtype=torch.float16, device="cuda"))
    assert PF.device_status() == 0



def test_residual_block_as_one_launch():
    """A ResidualBlock whose shortcut rides in conv2's launch (BatchNorm scales folded into fp16
    weights) agrees with the block run as conv2 + shortcut + residual epilogue."""
    import pcengine_b200 as pce
    from pcengine_b200.minkunet import ResidualBlock
    coords = surface_cloud(23, 56, batch=2)
    for cin, cout in ((32, 64), (64, 64)):
        torch.manual_seed(cin)
        block = ResidualBlock(cin, cout)
        pce.randomize_batchnorm(block, 9)
        block = block.half().cuda().eval()
        feats = torch.randn(len(coords), cin).half().cuda()
        outs = []
        for one in (True, False):
            block.one_kernel_tail = one
            x = pce.spTensor(feats, torch.from_numpy(coords).cuda(), None, [0, 0, 0], cmax_of(coords), init_tag=["auto"])
            with torch.no_grad():
                outs.append(block(x).feats.float().cpu())
        assert co.rel_l2(outs[0], outs[1]) <= 2e-3


def test_dense_product_on_tensor_cores():
    """1x1x1 layers with tensor-core friendly widths run the tcgen05 kernel in identity mode."""
    import pcengine_b200 as pce
    coords = random_cloud(6, 24, 5000)
    feats = torch.randn(len(coords), 192).half()
    x = _tensor(pce, coords, feats)
    lin = pce.conv3d(192, 128, 1, bias=True).cuda().half()
    y = lin(x)
    ref = co.pointwise_conv(feats, lin.kernel.detach().cpu(), lin.bias.detach().cpu())
    assert co.rel_l2(y.feats.float().cpu(), ref) <= 1e-3


@pytest.mark.parametrize("ks,world", [(3, 2), (5, 4)])
def test_slab_decomposition_matches_whole_scene(ks, world):
    """x-slabs with a kernel-radius halo (ranks emulated one after the other on this GPU): the owned
    rows of every slab are bit-identical to the rows of the undivided scene."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    from pcengine_b200 import multigpu as mg
    coords = surface_cloud(41, 96, batch=1)
    radius = (ks - 1) // 2
    torch.manual_seed(8)
    feats = torch.randn(len(coords), 64).half().cuda()
    w = (torch.randn(ks ** 3, 64, 64) / 40).half().cuda()
    cmax = cmax_of(coords)
    full_map = pce.KernelMap(torch.from_numpy(coords).cuda(), (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
    full = PF.conv_forward(feats, w, full_map.csr())
    cuts, owned = mg.split_scene(coords, world, radius)
    x = coords[:, 1]
    for g in range(world):
        halo = np.nonzero(((x >= cuts[g] - radius) & (x < cuts[g])) | ((x >= cuts[g + 1]) & (x < cuts[g + 1] + radius)))[0]
        rows = np.concatenate([owned[g], halo])
        local = torch.from_numpy(coords[rows]).cuda()
        km = pce.KernelMap(local, (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
        out = PF.conv_forward(feats[torch.from_numpy(rows).cuda()], w, km.csr())
        assert torch.equal(out[: len(owned[g])], full[torch.from_numpy(owned[g]).cuda()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("cin,cout", [(16, 16), (64, 64), (96, 32), (24, 19)])
def test_explicit_dataflow_d1(dtype, cin, cout):
    """Tag 'D1' runs gather -> per-offset GEMM (tensor cores for fp16 widths that allow it) -> scatter,
    for submanifold, strided and transposed layers; same numbers as the oracle, bit-identical run to run."""
    import pcengine_b200 as pce
    coords = surface_cloud(33, 60, batch=2)
    torch.manual_seed(9)
    feats = torch.randn(len(coords), cin).to(dtype)
    x = _tensor(pce, coords, feats, tags=("D1", "D1", "end"))
    conv = pce.conv3d(cin, cout, 3, bias=True).cuda().to(dtype)
    y = conv(x)
    km = x.kmaps[(conv.kernel_size_code, x.stride, conv.stride_code)]
    assert km.dataflow == "D1"
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    ref = co.conv_forward(feats, conv.kernel.detach().cpu(), d2, bias=conv.bias.detach().cpu())
    tol = TOL[dtype]
    assert co.rel_l2(y.feats.float().cpu(), ref) <= tol
    assert torch.equal(conv(x).feats, y.feats)
    down = pce.conv3d(cout, cin, 2, 2).cuda().to(dtype)
    up = pce.conv3d(cin, cout, 2, 2, transposed=True).cuda().to(dtype)
    z = down(y)
    u = up(z)
    d2s = ko.build_d2(coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], cmax_of(coords), False)
    refz = co.conv_forward(y.feats.cpu(), down.kernel.detach().cpu(), d2s)
    assert co.rel_l2(z.feats.float().cpu(), refz) <= tol
    refu = co.conv_forward(z.feats.cpu(), up.kernel.detach().cpu(), d2s, transposed=True)
    assert co.rel_l2(u.feats.float().cpu(), refu) <= tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_empty_and_tiny_tensors(dtype):
    """Zero voxels, one voxel and voxels without neighbours go through the same operators: an empty
    tensor stays empty with the right width, a lone voxel only sees the centre weight."""
    import pcengine_b200 as pce
    conv = pce.conv3d(16, 32, 3).cuda().to(dtype)
    down = pce.conv3d(32, 32, 2, 2).cuda().to(dtype)
    up = pce.conv3d(32, 16, 2, 2, transposed=True).cuda().to(dtype)
    for coords in (np.zeros((0, 4), np.int32), np.array([[0, 5, 5, 5]], np.int32),
                   np.array([[0, 0, 0, 0], [0, 9, 9, 9], [1, 0, 0, 0], [1, 20, 3, 7]], np.int32)):
        n = len(coords)
        feats = torch.randn(n, 16).to(dtype)
        x = pce.spTensor(feats.cuda(), torch.from_numpy(coords).cuda(), None, [0, 0, 0], [31, 31, 31], init_tag=["auto"])
        y = conv(x)
        assert y.feats.shape == (n, 32)
        z = down(y)
        u = up(z)
        assert u.feats.shape == (n, 16) and z.feats.shape[1] == 32
        if n:
            want = feats.float() @ conv.kernel.detach().float().cpu()[13]  # isolated voxels: the centre offset only
            assert co.rel_l2(y.feats.float().cpu(), want) <= TOL[dtype]
            d2 = ko.build_d2(coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], [31, 31, 31], False)
            assert np.array_equal(z.coords.cpu().numpy(), d2["out_coords"])


def test_negative_coordinates_and_large_batch_index():
    """Coordinates below zero (with matching bounds) and a batch index in the hundreds pack into the
    64-bit keys like any other; maps and features match the oracle."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    rng = np.random.default_rng(8)
    xyz = rng.integers(-12, 13, (4000, 3))
    coords = np.unique(np.concatenate([rng.choice([0, 7, 300], (4000, 1)), xyz], axis=1), axis=0).astype(np.int32)
    cmin, cmax = [-12, -12, -12], [12, 12, 12]
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), cmin, cmax, True)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (3, 3, 3), (1, 1, 1), (0, 0, 0), cmin, cmax, True)
    assert np.array_equal(km.map.cpu().numpy(), d2["map"].reshape(-1))
    feats = torch.randn(len(coords), 32).half()
    w = (torch.randn(27, 32, 32) / 30).half()
    out = PF.conv_forward(feats.cuda(), w.cuda(), km.csr())
    assert co.rel_l2(out.float().cpu(), co.conv_forward(feats, w, d2)) <= 1e-3
    ds = ko.build_d2(coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), cmin, cmax, False)  # derives the output bound
    kd = pce.KernelMap(torch.from_numpy(coords).cuda(), (2, 2, 2), (2, 2, 2), (0, 0, 0), cmin, ds["cmax_out"], False)
    assert np.array_equal(kd.out_coords.cpu().numpy(), ds["out_coords"])
    assert np.array_equal(kd.map.cpu().numpy(), ds["map"].reshape(-1))


def test_bias_keeps_the_second_operand_of_the_epilogue():
    """conv3d(bias=True) called with an epilogue that carries a second operand (a block's shortcut):
    the bias folds into the shift and the second operand still joins the sum."""
    import pcengine_b200 as pce
    from pcengine_b200.functional import FusedEpilogue
    coords = surface_cloud(71, 40)
    torch.manual_seed(4)
    feats = torch.randn(len(coords), 32).half()
    extra = torch.randn(len(coords), 16).half()
    w2 = (torch.randn(16, 32) / 4).half()
    scale = (0.5 + torch.rand(32)).float()
    conv = pce.conv3d(32, 32, 3, bias=True).cuda().half()
    x = _tensor(pce, coords, feats)
    ep = FusedEpilogue(scale=scale.cuda(), act="relu", extra_feats=extra.cuda(), extra_weight=w2.cuda())
    y = conv(x, epilogue=ep)
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    acc = co.conv_forward(feats, conv.kernel.detach().cpu(), d2) + extra.float() @ w2.float()
    want = torch.relu((acc + conv.bias.detach().float().cpu()) * scale)
    assert co.rel_l2(y.feats.float().cpu(), want) <= 1e-3


def test_weights_rewritten_through_data_need_invalidate_packed():
    """The tensor-core layout of a weight tensor is cached on it; a write through ``.data`` does not
    advance the version the cache is keyed on, so ``invalidate_packed`` is part of that recipe."""
    import pcengine_b200 as pce
    coords = surface_cloud(72, 40)
    torch.manual_seed(5)
    feats = torch.randn(len(coords), 64).half()
    conv = pce.conv3d(64, 64, 3).cuda().half()
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    y0 = conv(_tensor(pce, coords, feats)).feats.clone()
    new_w = (torch.randn(27, 64, 64) / 40).half()
    conv.kernel.data.copy_(new_w.cuda())
    pce.invalidate_packed(conv)
    y1 = conv(_tensor(pce, coords, feats)).feats
    assert co.rel_l2(y1.float().cpu(), co.conv_forward(feats, new_w, d2)) <= 1e-3
    assert not torch.equal(y0, y1)
    conv.reset_parameters()  # rewrites through .data and drops the cached layout itself
    y2 = conv(_tensor(pce, coords, feats)).feats
    assert co.rel_l2(y2.float().cpu(), co.conv_forward(feats, conv.kernel.detach().cpu(), d2)) <= 1e-3


def test_auto_tag_selects_the_measured_dataflow():
    """Tag 'auto': a wide fp16 layer on a small, very sparse map runs the explicit dataflow (the one
    cell of the sweep where it is faster), a dense neighbourhood or a narrow layer the fused one; both
    give the oracle's features."""
    import pcengine_b200 as pce
    rng = np.random.default_rng(77)
    lin = rng.choice(80 ** 3, 6000, replace=False)   # ~1% occupancy: hardly any neighbours
    sparse = np.stack([np.zeros_like(lin), lin // 6400, (lin // 80) % 80, lin % 80], 1).astype(np.int32)
    dense = surface_cloud(78, 40)
    torch.manual_seed(6)
    for coords, c, want_flow in ((sparse, 256, "D1"), (dense, 256, "D2"), (sparse, 64, "D2")):
        feats = torch.randn(len(coords), c).half()
        conv = pce.conv3d(c, c, 3).cuda().half()
        x = _tensor(pce, coords, feats, tags=("auto",))
        y = conv(x)
        km = x.kmaps[(conv.kernel_size_code, x.stride, conv.stride_code)]
        assert km.dataflow == want_flow, (len(coords), c, km.dataflow)
        d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
        assert co.rel_l2(y.feats.float().cpu(), co.conv_forward(feats, conv.kernel.detach().cpu(), d2)) <= 1e-3


def _split_layer_case(cin, cout, n_side, ks, stream_k):
    import pcengine_b200 as pce
    from pcengine_b200 import _lib
    from pcengine_b200 import functional as PF
    coords = surface_cloud(200 + n_side, n_side, batch=2)
    n = len(coords)
    subm = ks != 2
    d2 = ko.build_d2(coords, (ks,) * 3, (1, 1, 1) if subm else (2, 2, 2), (0, 0, 0), [0, 0, 0], cmax_of(coords), subm)
    km = pce.KernelMap(torch.from_numpy(coords).cuda(), (ks,) * 3, (1, 1, 1) if subm else (2, 2, 2), (0, 0, 0), [0, 0, 0],
                       d2["cmax_out"], subm)
    csr = km.csr()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    parts = _lib.lib.pce_conv_split_parts(csr.n_rows, n, cin, cout, ks ** 3, sms)
    scratch = _lib.lib.pce_conv_split_scratch_bytes(csr.n_rows, n, cin, cout, ks ** 3, sms)
    if stream_k:
        assert parts == 1 and scratch > 0, "the case is meant to be cut into shares of stages"
    else:
        assert parts > 1 and scratch == parts * csr.n_rows * cout * 4, "the case is meant to be split into parts"
    g = torch.Generator().manual_seed(cin + cout + n_side)
    x = torch.randn(n, cin, generator=g).half()
    w = (torch.randn(ks ** 3, cin, cout, generator=g) / (ks ** 3 * cin) ** 0.5).half()
    scale, shift = torch.rand(cout, generator=g) + 0.5, torch.randn(cout, generator=g)
    res = torch.randn(csr.n_rows, cout, generator=g).half()
    want = co.conv_forward(x, w, d2)
    eps = [None, PF.FusedEpilogue(scale=scale.cuda(), shift=shift.cuda(), residual=res.cuda(), act="leaky", slope=0.2)]
    wants = [want, torch.nn.functional.leaky_relu(want * scale + shift + res.float(), 0.2)]
    if subm:
        x2 = torch.randn(n, 64, generator=g).half()
        w2 = (torch.randn(64, cout, generator=g) / 8).half()
        eps.append(PF.FusedEpilogue(shift=shift.cuda(), act="relu", extra_feats=x2.cuda(), extra_weight=w2.cuda()))
        wants.append(torch.relu(want + x2.float() @ w2.float() + shift))
    for ep, ref in zip(eps, wants):
        a = PF.conv_forward(x.cuda(), w.cuda(), csr, ep)
        b = PF.conv_forward(x.cuda(), w.cuda(), csr, ep)
        assert torch.equal(a, b)
        assert co.rel_l2(a.float().cpu(), ref) <= 1e-3
        PF.SPLIT_TILES = False
        try:
            whole = PF.conv_forward(x.cuda(), w.cuda(), csr, ep)
        finally:
            PF.SPLIT_TILES = True
        assert co.rel_l2(a.float().cpu(), whole.float().cpu()) <= 5e-4  # same products, another fp32 association
    assert PF.device_status() == 0


@pytest.mark.split_tiles
@pytest.mark.parametrize("cin,cout,n_side,ks", [(256, 256, 20, 3), (128, 256, 30, 3), (96, 96, 48, 3), (128, 128, 26, 5), (256, 128, 24, 2)])
def test_small_maps_split_over_several_ctas(cin, cout, n_side, ks):
    """A map with few 128-row tiles runs with several CTAs per tile: every CTA takes a part of the tile's
    stage list, the fp32 partial sums are added in order by a second kernel that also applies the epilogue
    (scale, shift, residual or second operand, activation).  Same features as the oracle and as the unsplit
    kernel within fp16 rounding, bit-identical run to run."""
    _split_layer_case(cin, cout, n_side, ks, stream_k=False)


@pytest.mark.split_tiles
@pytest.mark.parametrize("cin,cout,n_side,ks", [(256, 256, 128, 3), (192, 96, 150, 3), (384, 256, 110, 3), (64, 64, 140, 3)])
def test_mid_size_maps_cut_into_equal_shares_of_stages(cin, cout, n_side, ks):
    """A map of half a wave to one wave of tiles with long stage chains is cut into equal shares of ring stages, one share per CTA slot,
    wherever the cuts fall inside the tiles; tiles that two or more CTAs worked on are summed in CTA order
    and finished by a second kernel.  Same checks as for the split into parts."""
    _split_layer_case(cin, cout, n_side, ks, stream_k=True)


def test_push_rows_gathers_into_consecutive_rows():
    """pce_push_rows (the halo mailbox's store kernel) on local memory: selected rows of a row-pitched matrix land
    in consecutive rows of the destination; without a row list it is a row-wise copy; rows that are not a
    multiple of 16 bytes are refused."""
    from pcengine_b200 import _lib
    g = torch.Generator().manual_seed(9)
    wide = torch.randn(300, 48, generator=g).half().cuda()
    src = wide[:, 8:40]                                   # 32 channels inside a 48-channel matrix: pitch 96 B
    rows = torch.tensor([5, 0, 299, 17, 17, 123], dtype=torch.int32, device="cuda")
    dst = torch.zeros(8, 64, dtype=torch.float16, device="cuda")
    st = _lib.stream_ptr(src.device)
    _lib.check(_lib.lib.pce_push_rows(src.data_ptr(), 96, rows.data_ptr(), 6, 64, dst.data_ptr(), 128, st), "pce_push_rows")
    assert torch.equal(dst[:6, :32], src[rows.long()]) and not dst[6:].any() and not dst[:, 32:].any()
    _lib.check(_lib.lib.pce_push_rows(src.data_ptr(), 96, None, 8, 64, dst.data_ptr(), 128, st), "pce_push_rows")
    assert torch.equal(dst[:, :32], src[:8])
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.pce_push_rows(src.data_ptr(), 96, None, 8, 24, dst.data_ptr(), 128, st), "pce_push_rows")
    assert _lib.lib.pce_push_rows(src.data_ptr(), 96, None, 0, 64, dst.data_ptr(), 128, st) == 0
