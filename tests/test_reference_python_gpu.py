"""The reference's OWN Python operator layer (script/spconv.py, script/sptensor.py, unmodified) running on
this library: ``PCEngine.backend`` is aliased to ``pcengine_b200.backend`` exactly as INTEGRATION.md shows, a
stub stands in for the ``open3d`` import of script/utils.py:2 (file reading, not on the path), and the
reference's ``conv3d`` modules are run and compared with the oracle.

The operator layer is taken from the reference tree when it is on this machine, else from its byte-compiled
image under oracle/_ref/script (written and loaded by oracle/build_ref.py); the tests skip when neither is there.
"""
import importlib
import importlib.util
import os
import sys
import types

import numpy as np
import pytest
import torch

from oracle import conv_oracle as co
from oracle import kmap_oracle as ko
from tests.helpers import cmax_of, random_cloud, surface_cloud

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_script_root():
    tree = os.environ.get("PCE_REFERENCE_TREE", "/root/reference")
    if os.path.exists(os.path.join(tree, "script", "spconv.py")):
        return tree, "source"
    image = os.path.join(ROOT, "oracle", "_ref")
    if os.path.exists(os.path.join(image, "script", "spconv.code")):
        return image, "image"
    return None, None


@pytest.fixture(scope="module")
def ref():
    """script.spconv / script.sptensor of the reference, bound to this library's backend module."""
    root, kind = _reference_script_root()
    if root is None:
        pytest.skip("neither the reference tree nor oracle/_ref/script is on this machine")
    import pcengine_b200.backend as backend
    names = ("PCEngine", "PCEngine.backend", "open3d")
    saved = {k: sys.modules.get(k) for k in names}
    pkg = types.ModuleType("PCEngine")
    pkg.backend = backend
    sys.modules["PCEngine"] = pkg
    sys.modules["PCEngine.backend"] = backend
    if "open3d" not in sys.modules:
        sys.modules["open3d"] = types.ModuleType("open3d")
    for k in [k for k in sys.modules if k == "script" or k.startswith("script.")]:
        del sys.modules[k]
    try:
        if kind == "source":
            sys.path.insert(0, root)
            try:
                importlib.import_module("script.spconv")
            finally:
                sys.path.remove(root)
        else:
            spec = importlib.util.spec_from_file_location("pce_b200_build_ref", os.path.join(ROOT, "oracle", "build_ref.py"))
            build_ref = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(build_ref)
            build_ref.load_reference_script(root)
        spconv, sptensor = sys.modules["script.spconv"], sys.modules["script.sptensor"]
        assert spconv.mapping_d2_cuda is backend.mapping_d2_cuda
        yield types.SimpleNamespace(conv3d=spconv.conv3d, spTensor=sptensor.spTensor)
    finally:
        for k in [k for k in sys.modules if k == "script" or k.startswith("script.")]:
            del sys.modules[k]
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def _tensor(ref, coords, feats, tags, dev):
    return ref.spTensor(coords=torch.from_numpy(coords).to(dev), feats=feats.to(dev), batchsize=int(coords[:, 0].max()) + 1,
                        buffer=torch.zeros(1, dtype=feats.dtype, device=dev), init_tag=list(tags),
                        coords_min=[0, 0, 0], coords_max=cmax_of(coords))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,cin,cout,tol", [(torch.float32, 16, 16, 1e-5), (torch.float32, 32, 64, 1e-5),
                                                (torch.float16, 64, 64, 1e-3)])
def test_reference_conv3d_submanifold_on_this_backend(ref, dtype, cin, cout, tol):
    dev = torch.device("cuda")
    coords = surface_cloud(401, 36, batch=2)
    g = torch.Generator().manual_seed(5)
    feats = torch.randn(len(coords), cin, generator=g).to(dtype)
    conv = ref.conv3d(cin, cout, 3, 1).to(dev).to(dtype)
    x = _tensor(ref, coords, feats, ["D2", "D2", "end"], dev)
    y = conv(x)
    torch.cuda.synchronize()
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    kmap = x.kmaps[(conv.kernel_size_code, x.stride, conv.stride_code)]
    assert np.array_equal(kmap[0].cpu().numpy().ravel(), d2["imap"]) and np.array_equal(kmap[1].cpu().numpy().ravel(), d2["omap"])
    assert np.array_equal(kmap[2].cpu().numpy(), d2["kpos"]) and np.array_equal(kmap[3].cpu().numpy(), d2["qkpos"])
    assert y.coords is x.coords
    want = co.conv_forward(feats, conv.kernel.detach().cpu(), d2)
    assert co.rel_l2(y.feats.float().cpu(), want) <= tol
    # the cached kernel map serves a second layer at the same resolution without a new build
    conv2 = ref.conv3d(cout, cin, 3, 1).to(dev).to(dtype)
    z = conv2(y)
    assert len(z.kmaps) == 1 and z.init_tag == ["D2", "end"]
    want2 = co.conv_forward(y.feats.cpu(), conv2.kernel.detach().cpu(), d2)
    assert co.rel_l2(z.feats.float().cpu(), want2) <= tol


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 1e-3)])
def test_reference_strided_then_transposed_on_this_backend(ref, dtype, tol):
    dev = torch.device("cuda")
    coords = random_cloud(402, 24, 3000, batch=2)
    g = torch.Generator().manual_seed(6)
    feats = torch.randn(len(coords), 32, generator=g).to(dtype)
    stem = ref.conv3d(32, 32, 3, 1).to(dev).to(dtype)
    down = ref.conv3d(32, 64, 3, 2, padding=1, bias=True).to(dev).to(dtype)
    up = ref.conv3d(64, 32, 3, 2, padding=1, transposed=True).to(dev).to(dtype)
    x = _tensor(ref, coords, feats, ["D2", "D2", "end"], dev)
    # the reference's transposed layer reads the fine coordinates from cbook[fine stride], which only a layer
    # whose OUTPUT has that stride registers (script/spconv.py:309,384): a network starts with such a layer
    feats = stem(x).feats.detach().cpu()
    x.feats = feats.to(dev)
    y = down(x)
    u = up(y)
    torch.cuda.synchronize()
    d2 = ko.build_d2(coords, (3, 3, 3), (2, 2, 2), (1, 1, 1), [0, 0, 0], cmax_of(coords), False)
    assert np.array_equal(y.coords.cpu().numpy(), d2["out_coords"])
    want = co.conv_forward(feats, down.kernel.detach().cpu(), d2, bias=down.bias.detach().cpu())
    assert co.rel_l2(y.feats.float().cpu(), want) <= tol
    want_u = co.conv_forward(y.feats.cpu(), up.kernel.detach().cpu(), d2, transposed=True)
    assert u.feats.shape[0] == len(coords) and u.coords is x.coords
    assert co.rel_l2(u.feats.float().cpu(), want_u) <= tol


@pytest.mark.gpu
def test_reference_gather_mm_scatter_tag_on_this_backend(ref):
    """init_tag 'D1': the reference allocates kv (not kv+1) kpos entries and grows the buffer itself."""
    dev = torch.device("cuda")
    coords = surface_cloud(403, 30)
    g = torch.Generator().manual_seed(7)
    feats = torch.randn(len(coords), 32, generator=g)
    conv = ref.conv3d(32, 32, 3, 1).to(dev)
    x = _tensor(ref, coords, feats, ["D1", "end"], dev)
    y = conv(x)
    torch.cuda.synchronize()
    d2 = ko.build_d2(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax_of(coords), True)
    want = co.conv_forward(feats, conv.kernel.detach().cpu(), d2)
    assert co.rel_l2(y.feats.float().cpu(), want) <= 1e-5
