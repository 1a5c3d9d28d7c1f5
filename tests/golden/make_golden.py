"""Generates the committed golden fixtures from the CPU oracle (run from the repository root):

    python tests/golden/make_golden.py

Each .npz holds a small seeded case: input coordinates, layer geometry, every kernel-map artefact
(output coordinates, indicator map, knnz/kpos/qkpos, pair lists, CSR-coded D1 forms, bitmask CSR) and
fp32 reference features for seeded fp16-representable inputs and weights.  The oracle itself is pinned
against dense conv3d by tests/test_oracle_dense.py; these files freeze its output so that a change
in either the oracle or the CUDA path shows up as a diff against a stored answer.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import conv_oracle as co  # noqa: E402
from oracle import kmap_oracle as ko  # noqa: E402
from tests.helpers import cmax_of, random_cloud, surface_cloud  # noqa: E402

CASES = {
    "subm3_random": dict(coords=lambda: random_cloud(101, 16, 700, batch=2), ks=(3, 3, 3), stride=(1, 1, 1), pad=(0, 0, 0), cin=16, cout=16),
    "subm3_surface": dict(coords=lambda: surface_cloud(102, 28), ks=(3, 3, 3), stride=(1, 1, 1), pad=(0, 0, 0), cin=32, cout=64),
    "subm5_surface": dict(coords=lambda: surface_cloud(103, 20), ks=(5, 5, 5), stride=(1, 1, 1), pad=(0, 0, 0), cin=16, cout=16),
    "down2_s2": dict(coords=lambda: random_cloud(104, 18, 900, batch=2), ks=(2, 2, 2), stride=(2, 2, 2), pad=(0, 0, 0), cin=32, cout=64),
    "down3_s2_p1": dict(coords=lambda: surface_cloud(105, 24), ks=(3, 3, 3), stride=(2, 2, 2), pad=(1, 1, 1), cin=16, cout=32),
}


def build(name, spec):
    coords = spec["coords"]()
    subm = spec["stride"] == (1, 1, 1)
    d2 = ko.build_d2(coords, spec["ks"], spec["stride"], spec["pad"], [0, 0, 0], cmax_of(coords), subm)
    d1 = ko.build_d1(d2)
    nb = ko.neighbour_csr(d2)
    nbt = ko.neighbour_csr(d2, transposed=True)
    g = torch.Generator().manual_seed(sum(map(ord, name)) + 7)
    kv = d2["kv"]
    feats = torch.randn(len(coords), spec["cin"], generator=g).half()
    w = (torch.randn(kv, spec["cin"], spec["cout"], generator=g) / (kv * spec["cin"]) ** 0.5).half()
    out = co.conv_forward(feats, w, d2)
    back_w = (torch.randn(kv, spec["cout"], spec["cin"], generator=g) / (kv * spec["cout"]) ** 0.5).half()
    back = co.conv_forward(out.half(), back_w, d2, transposed=True)
    return dict(coords=coords, ks=np.array(spec["ks"]), stride=np.array(spec["stride"]), pad=np.array(spec["pad"]),
                subm=np.array(subm), out_coords=d2["out_coords"], map=d2["map"], knnz=d2["knnz"], kpos=d2["kpos"],
                qkpos=d2["qkpos"], imap=d2["imap"], omap=d2["omap"], icsr=d1["icsr"], imap_coded=d1["imap"],
                ocsr=d1["ocsr"], omap_coded=d1["omap"], mask=nb["mask"], rowptr=nb["rowptr"], nbr=nb["nbr"],
                mask_t=nbt["mask"], rowptr_t=nbt["rowptr"], nbr_t=nbt["nbr"],
                feats=feats.numpy(), weights=w.numpy(), out=out.numpy(), back_weights=back_w.numpy(), back=back.numpy())


if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    for name, spec in CASES.items():
        data = build(name, spec)
        np.savez_compressed(os.path.join(here, name + ".npz"), **data)
        print(name, "n_in", len(data["coords"]), "n_out", len(data["out_coords"]), "pairs", len(data["imap"]))
