"""CPU restatement of the MinkUNet-shaped network of pcengine_b200/minkunet.py
(TEST INFRASTRUCTURE ONLY; the reference ships no model, so this follows the product's
own definition layer by layer, on the oracle's maps and convolution).

Activations are rounded to the feature dtype after every layer (the product stores
fp16 between layers); all arithmetic is fp32.
"""
from __future__ import annotations

import numpy as np
import torch

from . import conv_oracle as co
from . import kmap_oracle as ko


class _Net:
    def __init__(self, sd, coords, act_dtype):
        self.sd = {k: v.detach().cpu() for k, v in sd.items()}
        self.act_dtype = act_dtype
        self.levels = [dict(coords=np.ascontiguousarray(coords, np.int32), cmax=coords[:, 1:].max(0).tolist())]
        self.subm = {}
        self.down = {}

    def _round(self, x):
        return x.to(self.act_dtype).float()

    def subm_map(self, lvl, ks=3):
        key = (lvl, ks)
        if key not in self.subm:
            L = self.levels[lvl]
            self.subm[key] = ko.build_d2(L["coords"], (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], L["cmax"], True)
        return self.subm[key]

    def down_map(self, lvl):
        if lvl not in self.down:
            L = self.levels[lvl]
            d2 = ko.build_d2(L["coords"], (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], L["cmax"], False)
            self.down[lvl] = d2
            if len(self.levels) == lvl + 1:
                self.levels.append(dict(coords=d2["out_coords"], cmax=d2["cmax_out"]))
        return self.down[lvl]

    def bn(self, x, p):
        sd = self.sd
        return co.batchnorm_eval(x, sd[p + ".weight"], sd[p + ".bias"], sd[p + ".running_mean"], sd[p + ".running_var"])

    def conv_bn_relu(self, x, p, lvl, kind):
        w = self.sd[p + ".conv.kernel"]
        if kind == "subm":
            y = co.conv_forward(x, w, self.subm_map(lvl))
        elif kind == "down":
            y = co.conv_forward(x, w, self.down_map(lvl))
        else:  # "up": from level lvl+1 to lvl
            y = co.conv_forward(x, w, self.down_map(lvl), transposed=True)
        return self._round(torch.relu(self.bn(y, p + ".bn")))

    def res_block(self, x, p, lvl):
        sd = self.sd
        m = self.subm_map(lvl)
        y = self._round(torch.relu(self.bn(co.conv_forward(x, sd[p + ".conv1.kernel"], m), p + ".bn1")))
        if (p + ".short_conv.kernel") in sd:
            sc = self._round(self.bn(co.pointwise_conv(x, sd[p + ".short_conv.kernel"]), p + ".short_bn"))
        else:
            sc = x
        y = self.bn(co.conv_forward(y, sd[p + ".conv2.kernel"], m), p + ".bn2")
        return self._round(torch.relu(y + sc))


WIDTHS = (32, 32, 64, 128, 256, 256, 128, 96, 96)


def parameter_shapes(in_channels: int = 4, num_classes: int = 19, cr: float = 1.0) -> dict:
    """Name -> shape of every entry of the network's state dict, written out from the architecture
    (stem, four encoder and four decoder stages, classifier) without importing the product package;
    tests/test_bench_cpu.py checks it against ``pcengine_b200.MinkUNet().state_dict()``."""
    cs = [int(cr * c) for c in WIDTHS]
    shapes = {}

    def bn(prefix, c):
        for name in ("weight", "bias", "running_mean", "running_var"):
            shapes[f"{prefix}.{name}"] = (c,)
        shapes[f"{prefix}.num_batches_tracked"] = ()

    def conv_bn(prefix, cin, cout, kv):
        shapes[f"{prefix}.conv.kernel"] = (kv, cin, cout)
        bn(f"{prefix}.bn", cout)

    def block(prefix, cin, cout):
        shapes[f"{prefix}.conv1.kernel"] = (27, cin, cout)
        bn(f"{prefix}.bn1", cout)
        shapes[f"{prefix}.conv2.kernel"] = (27, cout, cout)
        bn(f"{prefix}.bn2", cout)
        if cin != cout:
            shapes[f"{prefix}.short_conv.kernel"] = (cin, cout)
            bn(f"{prefix}.short_bn", cout)

    conv_bn("stem.0", in_channels, cs[0], 27)
    conv_bn("stem.1", cs[0], cs[0], 27)
    for i in range(4):
        conv_bn(f"down.{i}", cs[i], cs[i], 8)
        block(f"enc.{i}.0", cs[i], cs[i + 1])
        block(f"enc.{i}.1", cs[i + 1], cs[i + 1])
    skips = [cs[3], cs[2], cs[1], cs[0]]
    for i in range(4):
        conv_bn(f"up.{i}", cs[4 + i], cs[5 + i], 8)
        block(f"dec.{i}.0", cs[5 + i] + skips[i], cs[5 + i])
        block(f"dec.{i}.1", cs[5 + i], cs[5 + i])
    shapes["classifier.kernel"] = (cs[8], num_classes)
    shapes["classifier.bias"] = (num_classes,)
    return shapes


def forward(state_dict, coords: np.ndarray, feats: torch.Tensor, act_dtype=torch.float16, return_maps: bool = False):
    """Logits [N, classes] (fp32 values rounded to ``act_dtype``) of the network whose
    parameters are ``state_dict`` (keys as produced by pcengine_b200.minkunet.MinkUNet).  With
    ``return_maps`` also the kernel maps the pass built: {("subm", level): d2, ("down", level): d2}."""
    net = _Net(state_dict, coords, act_dtype)
    x = net._round(feats.float())
    x = net.conv_bn_relu(x, "stem.0", 0, "subm")
    x = net.conv_bn_relu(x, "stem.1", 0, "subm")
    skips = [x]
    for i in range(4):
        x = net.conv_bn_relu(x, f"down.{i}", i, "down")
        x = net.res_block(x, f"enc.{i}.0", i + 1)
        x = net.res_block(x, f"enc.{i}.1", i + 1)
        skips.append(x)
    for i in range(4):
        lvl = 3 - i
        x = net.conv_bn_relu(x, f"up.{i}", lvl, "up")
        x = torch.cat([x, skips[lvl]], dim=1)
        x = net.res_block(x, f"dec.{i}.0", lvl)
        x = net.res_block(x, f"dec.{i}.1", lvl)
    out = net._round(co.pointwise_conv(x, net.sd["classifier.kernel"], net.sd["classifier.bias"]))
    if return_maps:
        maps = {("subm", lvl): m for (lvl, _ks), m in net.subm.items()}
        maps.update({("down", lvl): m for lvl, m in net.down.items()})
        return out, maps
    return out
