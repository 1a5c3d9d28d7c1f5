"""Fixtures written by the REFERENCE project's own CUDA code (tests/golden/make_ref_golden.py, run on a
B200 against the reference's unmodified extension): the pin of the oracle, and through it of the CUDA path.

CPU: the oracle reproduces the reference's kernel-map artefacts bit for bit and its fp32 features to 1e-5.
GPU: the CUDA path does the same, through the C ABI and through the five ``PCEngine.backend`` names; where
the compiled reference extension is present (oracle/_ref, see oracle/build_ref.py) it is also run live.
"""
import glob
import importlib.util
import os

import numpy as np
import pytest
import torch

from oracle import conv_oracle as co
from oracle import kmap_oracle as ko
from tests.helpers import cmax_of, random_cloud

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "ref_*.npz")))
IDS = [os.path.basename(f)[:-4] for f in FILES]
MAP_KEYS = ("out_coords", "map", "knnz", "kpos", "qkpos")
TOL_FP32 = 1e-5   # fp32 features against the reference's fp32 CUDA-core kernels
TOL_FP16 = 1e-2   # the reference's fp16 kernels accumulate in fp16 with atomics (its own check uses rtol 1e-2)


def _geom(g):
    return tuple(int(v) for v in g["ks"]), tuple(int(v) for v in g["stride"]), tuple(int(v) for v in g["pad"]), bool(g["subm"])


def test_reference_fixtures_exist():
    assert len(FILES) >= 5


@pytest.mark.parametrize("path", FILES, ids=IDS)
def test_oracle_matches_the_reference(path):
    g = np.load(path)
    ks, stride, pad, subm = _geom(g)
    coords = g["coords"]
    d2 = ko.build_d2(coords, ks, stride, pad, [0, 0, 0], cmax_of(coords), subm)
    for key in MAP_KEYS:
        assert np.array_equal(d2[key], g[key]), key
    feats = torch.from_numpy(g["feats"].astype(np.float32))
    w = torch.from_numpy(g["weights"].astype(np.float32))
    out = co.conv_forward(feats, w, d2)
    assert co.rel_l2(out, torch.from_numpy(g["out"])) <= TOL_FP32
    assert co.rel_l2(out, torch.from_numpy(g["out_tf32"])) <= 1e-3
    assert co.rel_l2(out, torch.from_numpy(g["out_fp16"]).float()) <= TOL_FP16


def _codes(g):
    ks, stride, pad, subm = _geom(g)
    return ko.encode3(ks), ko.encode3(stride), ko.encode3(pad), ks[0] * ks[1] * ks[2], subm


def _run_backend(be, g, dtype, dev, tf32=False):
    """The fetch-on-demand calls of script/spconv.py:345-376,240-253 on backend module ``be``."""
    coords = torch.from_numpy(g["coords"]).to(dev)
    ksc, sc, pc, kv, subm = _codes(g)
    n = coords.shape[0]
    imap = -torch.ones(kv * n, dtype=torch.int, device=dev)
    knnz = torch.zeros(kv, dtype=torch.int, device=dev)
    kpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    qkpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    cm = [int(v) for v in g["cmax_out"]]
    out_coords = be.mapping_d2_cuda(coords, int(g["coords"][:, 0].max()) + 1, ksc, kv, 0, 0, sc, ko.encode3((1, 1, 1)), pc,
                                    0, 0, 0, cm[0], cm[1], cm[2], imap, knnz, kpos, qkpos, subm)
    dense = imap.clone()
    idx = torch.nonzero(imap != -1)
    omap = imap[idx]
    imap = (idx % n).int()
    qsum = int(qkpos[-1].cpu())
    feats = torch.from_numpy(g["feats"]).to(dev).to(dtype)
    w = torch.from_numpy(g["weights"]).to(dev).to(dtype)
    out = torch.zeros((out_coords.shape[0], w.shape[2]), dtype=dtype, device=dev)
    be.conv_fwd_d2_cuda(feats, w, ksc, qsum, out, kpos, qkpos, imap, omap, n == out_coords.shape[0], tf32)
    torch.cuda.synchronize()
    return dict(out_coords=out_coords, map=dense, knnz=knnz, kpos=kpos, qkpos=qkpos), out


@pytest.mark.gpu
@pytest.mark.parametrize("path", FILES, ids=IDS)
def test_cuda_path_matches_the_reference(path):
    import pcengine_b200 as pce
    from pcengine_b200 import backend as be
    from pcengine_b200 import functional as PF
    g = np.load(path)
    dev = torch.device("cuda")
    # through the drop-in names, called as the reference's operator layer calls them
    for dtype, key, tol in ((torch.float32, "out", TOL_FP32), (torch.float16, "out_fp16", TOL_FP16)):
        maps, out = _run_backend(be, g, dtype, dev)
        for k in MAP_KEYS:
            assert np.array_equal(maps[k].cpu().numpy(), g[k]), k
        assert co.rel_l2(out.float().cpu(), torch.from_numpy(g[key]).float()) <= tol
        if dtype == torch.float16:  # the fp32-accumulating kernel is closer to the fp32 answer than the reference's fp16 one
            assert co.rel_l2(out.float().cpu(), torch.from_numpy(g["out"])) <= 1e-3
    # through the C ABI's own map object and both convolution kernels
    ks, stride, pad, subm = _geom(g)
    km = pce.KernelMap(torch.from_numpy(g["coords"]).to(dev), ks, stride, pad, [0, 0, 0], [int(v) for v in g["cmax_out"]], subm)
    assert np.array_equal(km.out_coords.cpu().numpy(), g["out_coords"])
    assert np.array_equal(km.map.cpu().numpy(), g["map"])
    assert np.array_equal(km.kpos.cpu().numpy(), g["kpos"]) and np.array_equal(km.qkpos.cpu().numpy(), g["qkpos"])
    x32 = torch.from_numpy(g["feats"]).float().to(dev)
    w32 = torch.from_numpy(g["weights"]).float().to(dev)
    out = PF.conv_forward(x32, w32, km.csr())
    assert co.rel_l2(out.cpu(), torch.from_numpy(g["out"])) <= TOL_FP32
    out = PF.conv_forward(x32.half(), w32.half(), km.csr())
    assert co.rel_l2(out.float().cpu(), torch.from_numpy(g["out"])) <= 1e-3
    assert PF.device_status() == 0


def _reference_backend():
    path = os.path.join(ROOT, "oracle", "_ref", "PCEngine", "backend.so")
    if not os.path.exists(path):
        pytest.skip("the reference's compiled extension is not present (oracle/build_ref.py builds it where the reference tree is)")
    spec = importlib.util.spec_from_file_location("backend", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["subm3_c32", "subm3_c64", "down3_s2_p1_c32_64"])
def test_live_reference_against_oracle_and_cuda_path(case):
    """The reference's own extension, the oracle and this library on a cloud no fixture holds."""
    from pcengine_b200 import backend as be
    ref = _reference_backend()
    dev = torch.device("cuda")
    seed = {"subm3_c32": 301, "subm3_c64": 302, "down3_s2_p1_c32_64": 303}[case]
    coords = random_cloud(seed, 26, 4000, batch=2)
    strided = case.startswith("down")
    ks, stride, pad = (3, 3, 3), ((2, 2, 2) if strided else (1, 1, 1)), ((1, 1, 1) if strided else (0, 0, 0))
    cin, cout = {"subm3_c32": (32, 32), "subm3_c64": (64, 64), "down3_s2_p1_c32_64": (32, 64)}[case]
    cmax = cmax_of(coords)
    cmax_out = [(cmax[i] + 2 * pad[i] - (ks[i] - 1)) // stride[i] for i in range(3)] if strided else cmax
    gen = torch.Generator().manual_seed(seed)
    g = dict(coords=coords, ks=np.array(ks), stride=np.array(stride), pad=np.array(pad), subm=np.array(not strided),
             cmax_out=np.array(cmax_out), feats=torch.randn(len(coords), cin, generator=gen).half().numpy(),
             weights=(torch.randn(27, cin, cout, generator=gen) / (27 * cin) ** 0.5).half().numpy())
    d2 = ko.build_d2(coords, ks, stride, pad, [0, 0, 0], cmax, not strided)
    want = co.conv_forward(torch.from_numpy(g["feats"]), torch.from_numpy(g["weights"]), d2)
    for name, mod in (("reference", ref), ("pcengine_b200", be)):
        maps, out = _run_backend(mod, g, torch.float32, dev)
        for k in MAP_KEYS:
            assert np.array_equal(maps[k].cpu().numpy(), d2[k]), (name, k)
        assert co.rel_l2(out.cpu(), want) <= TOL_FP32, name
        _, out16 = _run_backend(mod, g, torch.float16, dev)
        assert co.rel_l2(out16.float().cpu(), want) <= (TOL_FP16 if name == "reference" else 1e-3), name
