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
