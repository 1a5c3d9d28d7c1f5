"""bench.py pieces that need no GPU: the synthetic batch and its sharding, the seeded weights both arms
share, the CPU arm on a reduced sample (threads bounded by the affinity mask, product package not
imported), and the refusal of the GPU arm to run without a CUDA device."""
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import bench
    return bench


def test_synthetic_batch_is_seeded_and_differs_per_rank():
    bench = _bench()
    c0, f0, s0 = bench.make_batch(0, 2)
    c0b, f0b, _ = bench.make_batch(0, 2)
    c1, _, s1 = bench.make_batch(1, 2)
    assert np.array_equal(c0, c0b) and bool((f0 == f0b).all())
    assert c0.dtype == np.int32 and c0.shape[1] == 4 and f0.shape == (len(c0), bench.IN_CHANNELS)
    assert sum(s0) == len(c0) and set(np.unique(c0[:, 0]).tolist()) == {0, 1}
    assert s0 != s1  # every rank has its own scans
    assert len(np.unique(c0, axis=0)) == len(c0)  # voxels are unique


def test_the_batch_is_sharded_over_the_ranks_without_overlap():
    bench = _bench()
    from pcengine_b200 import multigpu as mg
    for world in (1, 2, 4, 8, 3):
        shares = [bench.scans_for_rank(bench.BATCH_SCANS, r, world) for r in range(world)]
        assert sorted(sum(shares, [])) == list(range(bench.BATCH_SCANS))
        assert shares == [mg.scans_for_rank(bench.BATCH_SCANS, r, world) for r in range(world)]
    # a rank's shard holds the same scans as the undivided batch does (batch index renumbered from 0)
    whole, wf, sizes = bench.make_scans([0, 1])
    part, pf, _ = bench.make_scans([1])
    assert np.array_equal(part[:, 1:], whole[sizes[0]:, 1:]) and bool((pf == wf[sizes[0]:]).all())
    assert set(part[:, 0].tolist()) == {0}


def test_seeded_weights_follow_the_product_network_by_name():
    bench = _bench()
    import pcengine_b200 as pce
    from oracle import minkunet_oracle as mo
    model = pce.MinkUNet(bench.IN_CHANNELS, bench.NUM_CLASSES)
    shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()}
    assert shapes == {k: tuple(v) for k, v in mo.parameter_shapes(bench.IN_CHANNELS, bench.NUM_CLASSES).items()}
    a = bench.seeded_state_dict(shapes)
    b = bench.seeded_state_dict(dict(reversed(list(shapes.items()))))  # order of the names does not matter
    assert all(torch.equal(a[k], b[k]) for k in a)
    model.load_state_dict(a)  # strict: every name and shape fits
    assert float(a["stem.0.bn.running_var"].min()) >= 0.8 and a["classifier.bias"].abs().max() > 0


def test_cpu_arm_on_one_scan_stays_inside_its_cores_and_off_the_product():
    code = ("import sys, os, json; sys.path.insert(0, %r); import bench, torch;"
            "v, dt, cores, sample = bench.oracle_scans_per_s(0, 1, 0, n_scans=1);"
            "print(json.dumps(dict(v=v, dt=dt, cores=cores, sample=sample, threads=torch.get_num_threads(),"
            "allowed=len(os.sched_getaffinity(0)), product=('pcengine_b200' in sys.modules))))" % ROOT)
    allowed = sorted(os.sched_getaffinity(0))[:2]
    r = subprocess.run(["taskset", "-c", ",".join(map(str, allowed)), sys.executable, "-c", code],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    import json
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["v"] > 0 and out["dt"] > 0 and "1 scan" in out["sample"]
    assert out["allowed"] == len(allowed) and out["cores"] <= out["allowed"] and out["threads"] <= out["allowed"]
    assert out["product"] is False  # the CPU arm never loads the CUDA library


def test_gpu_arm_refuses_to_run_without_cuda():
    if torch.cuda.is_available():
        return  # on a GPU box the arm runs; its output is checked by the driver
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "0", "--lean"],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode != 0 and "CUDA" in (r.stderr + r.stdout)
    assert not [line for line in r.stdout.splitlines() if line.startswith("{")]  # no number without a GPU
