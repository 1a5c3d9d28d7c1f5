"""The allocation-free map builder gives exactly what the workspace-based one gives.

``pce_map_build_d2_noalloc`` exists for callers that may not allocate device memory while they
run (a fixed-memory perception loop on a vehicle, a host runtime that passes a plug-in only its
inputs and outputs): its hash table sits in an array inside the library.  The test drives both
entry points through the C ABI on the same inputs, twice in a row, so that the second call meets
the table the first one left behind, and on a second, smaller input so that stale slots beyond
the cleared part would show.  The file name sorts last on purpose: a run that stops at the first
failure has then already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.helpers import cmax_of, random_cloud, surface_cloud

pytestmark = pytest.mark.gpu


def _build(lib, _lib, coords_d, out_d, geom, kv, use_noalloc, want_out):
    n_in, n_out = coords_d.size(0), out_d.size(0)
    dev = coords_d.device
    # poison the outputs: neither entry point may rely on their initial contents
    bufs = dict(map=torch.full((kv * n_in,), 7, dtype=torch.int32, device=dev),
                knnz=torch.full((kv,), 7, dtype=torch.int32, device=dev),
                kpos=torch.full((kv + 1,), 7, dtype=torch.int32, device=dev),
                qkpos=torch.full((kv + 1,), 7, dtype=torch.int32, device=dev),
                map_out=torch.full((kv * n_out,), 7, dtype=torch.int32, device=dev) if want_out else None,
                status=torch.zeros((1,), dtype=torch.int32, device=dev))
    st = torch.cuda.current_stream().cuda_stream
    if use_noalloc:
        rc = lib.pce_map_build_d2_noalloc(coords_d.data_ptr(), n_in, out_d.data_ptr(), n_out, C.byref(geom),
                                          bufs["map"].data_ptr(), bufs["knnz"].data_ptr(), bufs["kpos"].data_ptr(),
                                          bufs["qkpos"].data_ptr(), _lib.ptr(bufs["map_out"]),
                                          bufs["status"].data_ptr(), st)
    else:
        ws = torch.empty((lib.pce_map_workspace_bytes(n_in, kv, n_out),), dtype=torch.uint8, device=dev)
        rc = lib.pce_map_build_d2(coords_d.data_ptr(), n_in, out_d.data_ptr(), n_out, C.byref(geom), ws.data_ptr(),
                                  ws.numel(), bufs["map"].data_ptr(), bufs["knnz"].data_ptr(),
                                  bufs["kpos"].data_ptr(), bufs["qkpos"].data_ptr(), _lib.ptr(bufs["map_out"]),
                                  bufs["status"].data_ptr(), st)
    assert rc == 0, lib.pce_strerror(rc)
    torch.cuda.synchronize()
    return {k: (None if v is None else v.cpu().numpy()) for k, v in bufs.items()}


def _same(a, b):
    for k in a:
        if a[k] is None:
            assert b[k] is None
        else:
            assert np.array_equal(a[k], b[k]), k


def test_noalloc_map_equals_workspace_map_on_consecutive_calls():
    from pcengine_b200 import _lib
    from pcengine_b200.kmap import make_geom
    lib = _lib.lib
    dev = torch.device("cuda:0")
    big = surface_cloud(17, 96, batch=2)      # ~15k rows
    small = random_cloud(23, 20, 900)         # reuses a table the bigger input filled
    for coords in (big, small, big):
        cd = torch.from_numpy(coords).to(dev)
        cmax = cmax_of(coords)
        # submanifold 3x3x3 (outputs are the inputs)
        g = make_geom((3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
        ref = _build(lib, _lib, cd, cd, g, 27, False, False)
        first = _build(lib, _lib, cd, cd, g, 27, True, False)
        second = _build(lib, _lib, cd, cd, g, 27, True, False)
        _same(ref, first)
        _same(ref, second)
        assert ref["status"][0] == 0 and ref["kpos"][-1] > 0
        # strided 2x2x2 / stride 2, with the transposed table
        cmax2 = [(c - 1) // 2 for c in cmax]
        g2 = make_geom((2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], cmax2, False)
        oc = torch.from_numpy(np.unique(np.concatenate([coords[:, :1], coords[:, 1:] // 2], 1), axis=0)).to(dev)
        ref = _build(lib, _lib, cd, oc, g2, 8, False, True)
        first = _build(lib, _lib, cd, oc, g2, 8, True, True)
        second = _build(lib, _lib, cd, oc, g2, 8, True, True)
        _same(ref, first)
        _same(ref, second)
        assert ref["kpos"][-1] == len(coords)  # every input has exactly one parent


def test_noalloc_leaves_device_memory_as_it_is_and_takes_its_full_capacity():
    """After set-up calls of both map kinds (which also let the runtime load every kernel the entry
    point launches), further calls change nothing in the device's free memory; 131072 rows, the
    stated limit, are accepted and give the workspace builder's map."""
    from pcengine_b200 import _lib
    from pcengine_b200.kmap import make_geom
    lib = _lib.lib
    dev = torch.device("cuda:0")
    n = 131072
    rng = np.random.default_rng(5)
    lin = rng.choice(96 ** 3, n, replace=False)
    coords = np.stack([np.zeros(n, np.int64), lin // (96 * 96), (lin // 96) % 96, lin % 96], 1).astype(np.int32)
    cd = torch.from_numpy(coords).to(dev)
    oc = torch.from_numpy(np.unique(np.concatenate([coords[:, :1], coords[:, 1:] // 2], 1), axis=0)).to(dev)
    g = make_geom((3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], [95, 95, 95], True)
    g2 = make_geom((2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], [47, 47, 47], False)
    st = torch.cuda.current_stream().cuda_stream
    outs = dict(map=torch.empty((27 * n,), dtype=torch.int32, device=dev), small=torch.empty((28,), dtype=torch.int32, device=dev),
                map2=torch.empty((8 * n,), dtype=torch.int32, device=dev), map2_out=torch.empty((8 * oc.size(0),), dtype=torch.int32, device=dev))
    knnz, kpos, qkpos = (torch.empty((28,), dtype=torch.int32, device=dev) for _ in range(3))

    def both_kinds():
        rc = lib.pce_map_build_d2_noalloc(cd.data_ptr(), n, cd.data_ptr(), n, C.byref(g), outs["map"].data_ptr(), knnz.data_ptr(),
                                          kpos.data_ptr(), qkpos.data_ptr(), None, None, st)
        assert rc == 0, lib.pce_strerror(rc)
        rc = lib.pce_map_build_d2_noalloc(cd.data_ptr(), n, oc.data_ptr(), oc.size(0), C.byref(g2), outs["map2"].data_ptr(),
                                          knnz.data_ptr(), kpos.data_ptr(), qkpos.data_ptr(), outs["map2_out"].data_ptr(), None, st)
        assert rc == 0, lib.pce_strerror(rc)
        torch.cuda.synchronize()

    both_kinds()  # set-up
    free0, _ = torch.cuda.mem_get_info(dev)
    for _ in range(3):
        both_kinds()
    free1, _ = torch.cuda.mem_get_info(dev)
    assert free1 == free0
    ref = _build(lib, _lib, cd, cd, g, 27, False, False)
    got = _build(lib, _lib, cd, cd, g, 27, True, False)
    _same(ref, got)


def test_noalloc_rejects_more_rows_than_its_table_holds():
    from pcengine_b200 import _lib
    from pcengine_b200.kmap import make_geom
    lib = _lib.lib
    dev = torch.device("cuda:0")
    n = 131072 + 1
    coords = torch.zeros((n, 4), dtype=torch.int32, device=dev)
    g = make_geom((3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], [1, 1, 1], True)
    one = torch.zeros((28,), dtype=torch.int32, device=dev)
    before = lib.pce_kernel_launches()
    rc = lib.pce_map_build_d2_noalloc(coords.data_ptr(), n, coords.data_ptr(), n, C.byref(g), coords.data_ptr(),
                                      one.data_ptr(), one.data_ptr(), one.data_ptr(), None, None,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 8 and b"capacity" in lib.pce_strerror(rc)
    assert lib.pce_kernel_launches() == before  # nothing was launched
