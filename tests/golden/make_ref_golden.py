"""Generates golden fixtures from the REFERENCE project's own CUDA code (needs a GPU).

    python oracle/build_ref.py                                   # where the reference tree is (no GPU needed)
    python tests/golden/make_ref_golden.py --out DIR [--time]    # on a machine with a GPU

The first step compiles the reference's unmodified extension into ``oracle/_ref/`` (see
``oracle/build_ref.py``).  This script loads that module and calls its fetch-on-demand path
exactly as the reference's operator layer does -- allocations of script/spconv.py:345-352, the
``mapping_d2_cuda`` call of :362-368, the indicator post-pass of :370-376 and the
``conv_fwd_d2_cuda`` call of :240-253 -- on small seeded clouds, and stores what came back:
``out_coords``, ``map``, ``knnz``, ``kpos``, ``qkpos`` (all deterministic in the reference) and the
fp32 output features (``tf32=False``; plus, for information, the TF32 and fp16 outputs, whose
summation order and accumulate type the reference leaves to atomics and fp16).

Cases are limited to what the reference computes correctly: submanifold 3x3x3 and strided
ks=3/stride=2 (padding 0 and 1).  Its gather-GEMM-scatter map builder (out-of-bounds ``kpos``
write), its ks == stride output-coordinate shortcut and odd ks >= 5 strided layers are left out.

The committed ``ref_*.npz`` files under tests/golden/ were written by this script on a B200;
tests/test_ref_golden.py checks the CPU oracle and the CUDA path against them.
``--time`` also times the reference's forward on LiDAR-shaped single layers and prints JSON.
"""
import argparse
import importlib.util
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests.helpers import cmax_of, random_cloud, surface_cloud  # noqa: E402

CODE_X, CODE_Y = 94273, 311  # script/utils.py:233-234


def code3(v):
    return CODE_X * v[0] + CODE_Y * v[1] + v[2]


def load_reference_backend():
    path = os.path.join(ROOT, "oracle", "_ref", "PCEngine", "backend.so")
    if not os.path.exists(path):
        raise SystemExit(f"{path} is missing: run oracle/build_ref.py where the reference tree is")
    spec = importlib.util.spec_from_file_location("backend", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


CASES = {
    "ref_subm3_c16": dict(coords=lambda: random_cloud(201, 24, 3000, batch=2), ks=3, stride=1, pad=0, cin=16, cout=16),
    "ref_subm3_c32_64": dict(coords=lambda: surface_cloud(202, 44, batch=2), ks=3, stride=1, pad=0, cin=32, cout=64),
    "ref_subm3_c64": dict(coords=lambda: random_cloud(203, 20, 2500, batch=1), ks=3, stride=1, pad=0, cin=64, cout=64),
    "ref_down3_s2_p0": dict(coords=lambda: random_cloud(204, 22, 2600, batch=2), ks=3, stride=2, pad=0, cin=32, cout=32),
    "ref_down3_s2_p1": dict(coords=lambda: surface_cloud(205, 40, batch=2), ks=3, stride=2, pad=1, cin=64, cout=32),
}


def reference_map(be, coords_dev, ks, stride, pad, cmax_in, batch):
    """script/spconv.py:331-376 for init_tag 'D2'."""
    n = coords_dev.shape[0]
    kv = ks ** 3
    subm = stride == 1
    dev = coords_dev.device
    imap = -torch.ones(kv * n, dtype=torch.int, device=dev)
    knnz = torch.zeros(kv, dtype=torch.int, device=dev)
    kpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    qkpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    cmax = list(cmax_in)
    if not subm:
        cmax = [(cmax_in[i] + 2 * pad - (ks - 1)) // stride for i in range(3)]
    out_coords = be.mapping_d2_cuda(coords_dev, batch, code3([ks] * 3), kv, 0, 0, code3([stride] * 3), code3([1, 1, 1]),
                                    code3([pad] * 3), 0, 0, 0, cmax[0], cmax[1], cmax[2], imap, knnz, kpos, qkpos, subm)
    torch.cuda.synchronize()
    dense = imap.clone()
    nonzero_idx = torch.nonzero(imap != -1)
    omap = imap[nonzero_idx]
    imap = (nonzero_idx % n).int()
    qsum = int(qkpos[-1].cpu())
    return dict(out_coords=out_coords, map=dense, knnz=knnz, kpos=kpos, qkpos=qkpos, imap=imap, omap=omap, qsum=qsum,
                subm=subm, cmax_out=cmax)


def reference_forward(be, feats, kernel, ks, m, tf32):
    """script/spconv.py:240-253 (not transposed); the output starts at zero as conv_d2 allocates it."""
    n_out = m["out_coords"].shape[0]
    out = torch.zeros((n_out, kernel.shape[2]), dtype=feats.dtype, device=feats.device)
    separate_mid = feats.shape[0] == n_out  # script/spconv.py:229
    be.conv_fwd_d2_cuda(feats, kernel, code3([ks] * 3), m["qsum"], out, m["kpos"], m["qkpos"], m["imap"], m["omap"],
                        separate_mid, tf32)
    torch.cuda.synchronize()
    return out


def make_case(be, name, spec):
    coords = spec["coords"]()
    dev = torch.device("cuda")
    ks, stride, pad = spec["ks"], spec["stride"], spec["pad"]
    batch = int(coords[:, 0].max()) + 1
    m = reference_map(be, torch.from_numpy(coords).to(dev), ks, stride, pad, cmax_of(coords), batch)
    g = torch.Generator().manual_seed(sum(map(ord, name)) + 11)
    kv = ks ** 3
    feats = torch.randn(len(coords), spec["cin"], generator=g).half().float()
    w = (torch.randn(kv, spec["cin"], spec["cout"], generator=g) / (kv * spec["cin"]) ** 0.5).half().float()
    out = reference_forward(be, feats.to(dev), w.to(dev), ks, m, False)
    out_tf32 = reference_forward(be, feats.to(dev), w.to(dev), ks, m, True)
    out_fp16 = reference_forward(be, feats.half().to(dev), w.half().to(dev), ks, m, False)
    return dict(coords=coords, ks=np.array([ks] * 3), stride=np.array([stride] * 3), pad=np.array([pad] * 3),
                subm=np.array(m["subm"]), cmax_out=np.array(m["cmax_out"]),
                out_coords=m["out_coords"].cpu().numpy(), map=m["map"].cpu().numpy(), knnz=m["knnz"].cpu().numpy(),
                kpos=m["kpos"].cpu().numpy(), qkpos=m["qkpos"].cpu().numpy(),
                feats=feats.numpy().astype(np.float16), weights=w.numpy().astype(np.float16),
                out=out.cpu().numpy(), out_tf32=out_tf32.cpu().numpy(), out_fp16=out_fp16.cpu().numpy())


def time_reference(be, reps=20):
    """Reference forward (fp16, fetch-on-demand, kernel map cached) on LiDAR-shaped single layers."""
    from pcengine_b200 import synth  # generator only
    dev = torch.device("cuda")
    coords = synth.with_batch(synth.lidar_scan(2000))
    cdev = torch.from_numpy(coords).to(dev)
    m = reference_map(be, cdev, 3, 1, 0, cmax_of(coords), 1)
    pairs = int(m["imap"].numel()) + len(coords)
    rows = []
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    for c in (32, 64, 128):
        feats = torch.randn(len(coords), c, device=dev).half()
        w = (torch.randn(27, c, c, device=dev) / (27 * c) ** 0.5).half()
        for _ in range(3):
            reference_forward(be, feats, w, 3, m, False)
        # the reference launches on the legacy default stream: time with events recorded there
        ts = []
        for _ in range(reps):
            flush.zero_()
            out = torch.zeros((len(coords), c), dtype=feats.dtype, device=dev)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(torch.cuda.default_stream()):
                e0.record()
                be.conv_fwd_d2_cuda(feats, w, code3([3] * 3), m["qsum"], out, m["kpos"], m["qkpos"], m["imap"], m["omap"], True, False)
                e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        us = ts[len(ts) // 2]
        byts = 2 * (2 * len(coords) * c) + 2 * 27 * c * c + 4 * pairs
        rows.append(dict(layer=f"subm3 {c}->{c} fp16", voxels=len(coords), pairs=pairs, us=round(us, 1),
                         gbs=round(byts / us / 1e3, 1), tflops=round(2 * pairs * c * c / us / 1e6, 2)))
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--time", action="store_true")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the reference has no CPU path: this script needs a CUDA device")
    be = load_reference_backend()
    os.makedirs(args.out, exist_ok=True)
    for name, spec in CASES.items():
        data = make_case(be, name, spec)
        np.savez_compressed(os.path.join(args.out, name + ".npz"), **data)
        print(name, "n_in", len(data["coords"]), "n_out", len(data["out_coords"]), "pairs", int(data["knnz"].sum()), flush=True)
    if args.time:
        print(json.dumps({"reference_on_gpu": time_reference(be)}))
