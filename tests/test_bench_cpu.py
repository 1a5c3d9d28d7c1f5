"""bench.py pieces that need no GPU: the synthetic batch, the CPU arm on a reduced sample, and the
refusal of the GPU arm to run without a CUDA device."""
import json
import os
import subprocess
import sys

import numpy as np

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


def test_cpu_arm_on_one_scan():
    bench = _bench()
    v, dt, cores, sample = bench.oracle_scans_per_s(0, 1, 0, n_scans=1)
    assert v > 0 and dt > 0 and cores >= 1 and "1 scan" in sample


def test_gpu_arm_refuses_to_run_without_cuda():
    import torch
    if torch.cuda.is_available():
        return  # on a GPU box the arm runs; its output is checked by the driver
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "0", "--lean"],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode != 0 and "CUDA" in (r.stderr + r.stdout)
    assert not [line for line in r.stdout.splitlines() if line.startswith("{")]  # no number without a GPU
