import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "split_tiles: runs with small maps split over several CTAs per tile (the default)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Layers on small maps are split over several CTAs per tile (fp32 partial sums added by a second kernel),
# which associates the fp32 sum differently from the one-CTA chain.  Tests that assert BIT-identity between
# schedules (tile heights, row orders, slabs vs whole scene, the two kernels) run with the split off, which is
# what they are about; parity tests against the oracle and the reference run the default, split, path, and
# tests marked `split_tiles` exercise it explicitly.
_SPLIT_ON_MODULES = {"test_baseline_configs_gpu", "test_ref_golden", "test_reference_python_gpu", "test_backend_dropin_gpu",
                     "test_golden"}


@pytest.fixture(autouse=True)
def _split_policy(request):
    if "gpu" not in request.keywords:
        yield
        return
    from pcengine_b200 import _lib
    from pcengine_b200 import functional as PF
    on = request.module.__name__.rsplit(".", 1)[-1] in _SPLIT_ON_MODULES or "split_tiles" in request.keywords
    PF.SPLIT_TILES = on
    _lib.lib.pce_tune(7, 1 if on else 0)
    try:
        yield
    finally:
        PF.SPLIT_TILES = True
        _lib.lib.pce_tune(7, 1)
