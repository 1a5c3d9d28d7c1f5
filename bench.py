"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched through torchrun)
    python bench.py --impl reference --gpus N --steps K --warmup W

Workload (``config.workload`` = "minkunet_lidar_batch8"): one step is one inference pass of the
MinkUNet-shaped network (fp16, seeded random weights) over THE batch of 8 synthetic 64-beam LiDAR
scans (seeds 2000..2007), kernel-map construction included.  With N GPUs the 8 scans are sharded
8/N per rank (a rank collates its share into one batch); no collective touches the data path, the
step time is the slowest rank's, ``scaling`` is "strong".  ``weak_scans_per_s`` (N > 1) is the same
loop with 8 scans of its own on every rank.

The single JSON line carries: the device-timed whole-job throughput with inputs resident in HBM
(``value``), the same metric through host buffers with the copies inside the timed region
(``e2e``), the roofline of the dominant convolution kernel from per-launch CUDA events, whether
the kernel maps and logits of the timed batch equal the CPU oracle's (``parity``; a line whose
parity fails carries ``value: null``), per-layer figures for the single-layer configurations
(``layers``: LiDAR layers with the reference's own CUDA kernels timed beside them when its compiled
extension is present, the 20k-voxel fp32 layer, the indoor sweep), the 1.5 M-voxel scene in x-slabs
across the ranks (``scene_slabs``), the CPU oracle timed on the host cores (``cpu_baseline``) and the
GPU clocks sampled during the run.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH_SCANS = 8          # the batch of 8 LiDAR scans the metric is quoted on
SCANS_PER_GPU = BATCH_SCANS  # scans per rank of the weak-scaling side figure
IN_CHANNELS = 4
NUM_CLASSES = 19
WEIGHT_SEED = 4001
METRIC = "minkunet_scans_per_s"
UNIT = "scans/s"
PARITY_TOL = 5e-3        # rel-L2 of the fp16 network's logits against the fp32-arithmetic oracle network


# ----------------------------------------------------------------------------- inputs
def _synth():
    """The seeded generators (NumPy only), loaded by file path: the CPU arm must not import the
    product package, whose import loads the CUDA library."""
    name = "pce_b200_synth_generators"
    if name not in sys.modules:
        import importlib.util
        spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "pcengine_b200", "synth.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules[name]


def make_scans(ids):
    """Collated int32 coords [N,4] and fp16 features [N,4] of the scans ``ids`` (scan i: LiDAR seed
    2000 + i, feature seed 9000 + i; batch index = position in ``ids``).  Host NumPy / torch."""
    synth = _synth()
    coords, feats, sizes = [], [], []
    for b, i in enumerate(ids):
        xyz = synth.lidar_scan(2000 + int(i))
        coords.append(synth.with_batch(xyz, b))
        g = torch.Generator().manual_seed(9000 + int(i))
        feats.append(torch.randn(len(xyz), IN_CHANNELS, generator=g).half())
        sizes.append(len(xyz))
    return np.concatenate(coords), torch.cat(feats), sizes


def make_batch(rank: int, n_scans: int = SCANS_PER_GPU):
    """The weak-scaling batch of ``rank``: ``n_scans`` scans of its own (ids 8*rank ...)."""
    return make_scans([SCANS_PER_GPU * rank + i for i in range(n_scans)])


def scans_for_rank(n_scans: int, rank: int, world: int):
    """Contiguous, balanced share of the batch for ``rank`` (same rule as pcengine_b200.multigpu)."""
    base, extra = divmod(n_scans, world)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def seeded_state_dict(shapes: dict, seed: int = WEIGHT_SEED, dtype=torch.float16) -> dict:
    """Network parameters by NAME (one generator per entry, seeded from the name): both arms build
    the identical weights from the names and shapes alone.  Convolution kernels and biases are
    U(+-1/sqrt(C_out*kv)) as ``conv3d.reset_parameters`` draws them (script/spconv.py:101-106);
    BatchNorm gets non-trivial affine terms and running statistics so the fused epilogues work."""
    import zlib
    out = {}
    for name, shape in shapes.items():
        shape = tuple(shape)
        g = torch.Generator().manual_seed((seed * 1000003 + zlib.crc32(name.encode())) % (1 << 62))
        prefix, leaf = name.rsplit(".", 1)
        is_bn = (prefix + ".running_mean") in shapes
        if leaf == "num_batches_tracked":
            t = torch.zeros(shape, dtype=torch.long)
        elif leaf == "kernel":
            kv = shape[0] if len(shape) == 3 else 1
            t = ((torch.rand(shape, generator=g) * 2 - 1) / (shape[-1] * kv) ** 0.5).to(dtype)
        elif is_bn and leaf in ("weight", "running_var"):
            t = (0.8 + 0.4 * torch.rand(shape, generator=g)).to(dtype)
        elif is_bn:
            t = ((torch.rand(shape, generator=g) - 0.5) * 0.2).to(dtype)
        else:  # a convolution's bias
            t = ((torch.rand(shape, generator=g) * 2 - 1) / shape[0] ** 0.5).to(dtype)
        out[name] = t
    return out


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, source="fallback")


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons every 50 ms while the timed regions run:
    through NVML in this process (a looping nvidia-smi child was measured to slow the timed loop by up
    to 25 %), falling back to nvidia-smi when the NVML binding is missing.  Read-only queries."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.nvml, self.samples, self.stop_flag, self.thread = None, [], threading.Event(), None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        reasons_of = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag.is_set():
            try:
                self.samples.append((n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM),
                                     n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM),
                                     int(reasons_of(self.handle))))
            except Exception:
                pass
            self.stop_flag.wait(0.05)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            if not self.samples:
                return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
            reasons = sorted(name for name, bit in self.BITS.items() if any(s[2] & bit for s in self.samples))
            return dict(sm_mhz=float(np.median([s[0] for s in self.samples])),
                        sm_max_mhz=float(max(s[1] for s in self.samples)), reasons=reasons, samples=len(self.samples),
                        source="nvml")
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["clock sampling unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        return dict(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm),
                    source="nvidia-smi")


# ----------------------------------------------------------------------------- CPU arm
def cpu_threads() -> int:
    """Host threads the CPU arm may use: the cores this process is allowed on, never more."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def oracle_pass(ids, steps: int, warmup: int, want_outputs: bool = False):
    """The CPU restatement (oracle network: NumPy maps + PyTorch CPU gather-matmul-scatter) on the
    scans ``ids`` collated into one batch, ``steps`` timed passes.  Imports nothing of the product.
    Returns (scans/s, s per pass, threads, sample text, logits, maps) -- the last two of the final pass
    when ``want_outputs``."""
    from oracle import minkunet_oracle as mo
    threads = cpu_threads()
    torch.set_num_threads(threads)
    coords, feats, sizes = make_scans(ids)
    sd = seeded_state_dict(mo.parameter_shapes(IN_CHANNELS, NUM_CLASSES))
    logits = maps = None
    for _ in range(warmup):
        mo.forward(sd, coords, feats)
    t0 = time.perf_counter()
    for _ in range(steps):
        res = mo.forward(sd, coords, feats, return_maps=want_outputs)
        if want_outputs:
            logits, maps = res
    dt = (time.perf_counter() - t0) / max(steps, 1)
    sample = f"{len(ids)} scan(s) of the batch ({sum(sizes)} voxels) per step, {steps} step(s) timed"
    return len(ids) / dt, dt, torch.get_num_threads(), sample, logits, maps


def oracle_scans_per_s(rank: int, steps: int, warmup: int, n_scans: int = SCANS_PER_GPU):
    v, dt, cores, sample, _, _ = oracle_pass(list(range(n_scans)), steps, warmup)
    return v, dt, cores, sample


def run_reference(args):
    """The CPU arm: the reference has no CPU implementation, so this is the oracle port on all host
    cores this process may use.  Rank 0 alone runs; it times exactly ``--steps`` steps, each over a
    sample of the batch sized (from one probe pass over one scan) so the run ends within minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    _, probe_dt, _, _, _, _ = oracle_pass([0], 1, 0)
    budget_s = 150.0
    n = int(budget_s / max(probe_dt * (steps + warmup), 1e-9))
    n = max(1, min(BATCH_SCANS, n))
    v, dt, cores, sample, _, _ = oracle_pass(list(range(n)), steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "minkunet_lidar_batch8", "note": "CPU oracle (NumPy maps + PyTorch CPU gather-matmul-scatter, "
                   "fp32 arithmetic on fp16 values): the reference has no CPU implementation", "sample": sample},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU arm
LAYERS = {  # name: (map kind, kv, c_in, c_out)
    "subm3_32x32": ("subm", 27, 32, 32), "subm3_64x64": ("subm", 27, 64, 64), "subm3_96x96": ("subm", 27, 96, 96),
    "subm3_128x128": ("subm", 27, 128, 128),
    "subm3_256x256": ("subm", 27, 256, 256), "down2s2_32x64": ("down", 8, 32, 64), "up2s2_64x32": ("up", 8, 64, 32),
}
DEFAULT_LAYERS = ["subm3_32x32", "subm3_64x64", "subm3_96x96", "subm3_128x128", "down2s2_32x64", "up2s2_64x32"]


def _host_lead():
    """Keeps the GPU busy for ~0.25 ms so that the host has queued the timed launch (and its event
    pair) before the GPU gets to it: a kernel-only time then holds no launch latency of an idle GPU."""
    torch.cuda._sleep(500000)


def _timed(fn, flush, iters: int, warmup: int) -> float:
    """Median device time (s) of ``fn`` between two events, L2 flushed before every run."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        _host_lead()
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b) * 1e-3)
    return float(np.median(ts))


def _conv_row(name, t, n_in, n_out, pairs, kv, cin, cout, esize, pk):
    by = esize * (n_in * cin + n_out * cout) + esize * kv * cin * cout + 4 * pairs
    fl = 2.0 * pairs * cin * cout
    return {"layer": name, "n_in": n_in, "n_out": n_out, "pairs": pairs, "us": t * 1e6,
            "GB/s": by / t / 1e9, "TFLOP/s": fl / t / 1e12, "hbm_frac": by / t / 1e9 / pk["hbm_gbs"],
            "tensor_frac": fl / t / 1e12 / pk["tflops"], "alg_bytes": by, "alg_flops": fl}


def _reference_extension():
    """The reference's own compiled CUDA extension (oracle/_ref, built by oracle/build_ref.py where the
    reference tree is), or None: a same-GPU comparator for the single layers, never part of the product path."""
    path = os.path.join(ROOT, "oracle", "_ref", "PCEngine", "backend.so")
    if not os.path.exists(path):
        return None
    try:
        import importlib.util
        spec = importlib.util.spec_from_file_location("backend", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    except Exception:
        return None


def _reference_subm3(ref, coords, cmax):
    """The reference's fetch-on-demand map of a submanifold 3x3x3 layer, built by its own
    mapping_d2_cuda with the allocations and post-pass of script/spconv.py:345-376."""
    n, kv, dev = coords.shape[0], 27, coords.device
    code = lambda v: 94273 * v[0] + 311 * v[1] + v[2]
    imap = -torch.ones(kv * n, dtype=torch.int, device=dev)
    knnz = torch.zeros(kv, dtype=torch.int, device=dev)
    kpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    qkpos = torch.zeros(kv + 1, dtype=torch.int, device=dev)
    ref.mapping_d2_cuda(coords, 1, code((3, 3, 3)), kv, 0, 0, code((1, 1, 1)), code((1, 1, 1)), code((0, 0, 0)), 0, 0, 0,
                        cmax[0], cmax[1], cmax[2], imap, knnz, kpos, qkpos, True)
    idx = torch.nonzero(imap != -1)
    omap = imap[idx]
    imap = (idx % n).int()
    return dict(kpos=kpos, qkpos=qkpos, imap=imap, omap=omap, qsum=int(qkpos[-1].cpu()), code=code((3, 3, 3)))


def layer_table(dev, pk, names=None, scans: int = 1, iters: int = 10, warmup: int = 3, with_reference: bool = False,
                level: int = 0):
    """Single LiDAR-shaped layers on ``scans`` collated scans (seeds 2000..): kernel-only time per layer
    with an L2 flush between launches; algorithmic bytes / flops per launch against the measured peaks.
    ``with_reference``: the reference's own fp16 kernels on the same submanifold layers, same timing.
    ``level``: run on the coordinates after that many 2x2x2 / stride-2 down-samplings (the deeper levels
    of the network: fewer, denser rows)."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords_h, _, _ = make_scans(list(range(scans)))
    coords = torch.from_numpy(coords_h).to(dev)
    cmax = coords_h[:, 1:].max(0).tolist()
    for _ in range(level):
        cmax = [(c - 1) // 2 for c in cmax]
        coords = pce.KernelMap(coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0], cmax, False).out_coords.contiguous()
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    names = list(names or DEFAULT_LAYERS)
    maps = {}
    ref = _reference_extension() if with_reference else None
    ref_map = None

    def csr_for(kind):
        if kind == "subm":
            if "subm" not in maps:
                maps["subm"] = pce.KernelMap(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
            return maps["subm"].csr()
        if "down" not in maps:
            maps["down"] = pce.KernelMap(coords, (2, 2, 2), (2, 2, 2), (0, 0, 0), [0, 0, 0],
                                         [(c - 1) // 2 for c in cmax], False)
        return maps["down"].csr(transposed=(kind == "up"))

    rows = []
    g = torch.Generator().manual_seed(5)
    for name in names:
        kind, kv, cin, cout = LAYERS[name]
        csr = csr_for(kind)
        x = torch.randn(csr.n_src, cin, generator=g).half().to(dev)
        w = (torch.randn(kv, cin, cout, generator=g) / (kv * cin) ** 0.5).half().to(dev)
        pairs = int(csr.rowptr[-1].item())
        t = _timed(lambda: PF.conv_forward(x, w, csr), flush, iters, warmup)
        row = _conv_row(name, t, csr.n_src, csr.n_rows, pairs, kv, cin, cout, 2, pk)
        if ref is not None and kind == "subm":
            # (the reference's ks == stride output-coordinate shortcut is inconsistent with its own query
            # kernel, so its 2x2x2 stride-2 layers are not run)
            if ref_map is None:
                ref_map = _reference_subm3(ref, coords, cmax)
            m = ref_map
            out = torch.empty((csr.n_rows, cout), dtype=torch.float16, device=dev)

            def ref_layer():  # what conv_d2.forward does per call: zero-filled output, then the kernels
                out.zero_()
                ref.conv_fwd_d2_cuda(x, w, m["code"], m["qsum"], out, m["kpos"], m["qkpos"], m["imap"], m["omap"], True, False)

            row["reference_us"] = _timed(ref_layer, flush, iters, warmup) * 1e6
            row["speedup_vs_reference_kernels"] = row["reference_us"] / row["us"]
        rows.append(row)
    return rows, int(coords.size(0))


def config1_row(dev, pk, iters: int = 10, warmup: int = 3):
    """The 20,000-voxel case: uniform sample of a 64^3 grid (seed 1001), submanifold 3x3x3, C 16 -> 16,
    fp32.  Kernel-map construction (hash insert, query, scans), the neighbour CSR and the convolution,
    each kernel-only with the L2 flushed."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    synth = _synth()
    coords_h = synth.with_batch(synth.uniform_grid(20000, 64, 1001))
    coords = torch.from_numpy(coords_h).to(dev)
    cmax = coords_h[:, 1:].max(0).tolist()
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    n, kv = len(coords_h), 27
    build = lambda: pce.KernelMap(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
    t_map = _timed(build, flush, iters, warmup)
    km = build()
    t_csr = _timed(lambda: (km._csr.clear(), km.csr()), flush, iters, warmup)
    csr = km.csr()
    pairs = int(csr.rowptr[-1].item())
    g = torch.Generator().manual_seed(1001)
    x = torch.randn(n, 16, generator=g).to(dev)
    w = (torch.randn(kv, 16, 16, generator=g) / (kv * 16) ** 0.5).to(dev)
    t = _timed(lambda: PF.conv_forward(x, w, csr), flush, iters, warmup)
    row = _conv_row("config1 subm3 16x16 fp32", t, n, n, pairs, kv, 16, 16, 4, pk)
    lookups = n * (kv - 1)
    map_bytes = 28 * n + 12 * lookups + 4 * n * kv
    row.update({"voxels": n, "map_us": t_map * 1e6, "csr_us": t_csr * 1e6, "map_lookups_per_s": lookups / t_map,
                "map_GB/s": map_bytes / t_map / 1e9, "map_hbm_frac": map_bytes / t_map / 1e9 / pk["hbm_gbs"]})
    return row


def indoor_rows(dev, pk, iters: int = 5, warmup: int = 2, both: bool = True):
    """The indoor-room sweep: one 8x8x3 m room voxelised at 2 cm (about 200 k voxels), submanifold
    3x3x3 at C_in = C_out in {16, 32, 64, 96, 128, 256}, fp16, kernel-only with an L2 flush between
    launches: what the 'auto' selector picks and, with ``both``, each dataflow."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    from pcengine_b200.spconv import _choose_dataflow
    synth = _synth()
    xyz, samples = synth.indoor_room(3001, 200000)
    coords = torch.from_numpy(synth.with_batch(xyz)).to(dev)
    km = pce.KernelMap(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], xyz.max(0).tolist(), True)
    csr = km.csr()
    pairs = int(csr.rowptr[-1].item())
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator().manual_seed(3)
    rows = []
    for c in (16, 32, 64, 96, 128, 256):
        x = torch.randn(km.n_in, c, generator=g).half().to(dev)
        w = (torch.randn(27, c, c, generator=g) / (27 * c) ** 0.5).half().to(dev)
        pick = _choose_dataflow("auto", c, c, pairs / km.n_in, km.n_in, torch.float16)
        fns = {"D2": lambda: PF.conv_forward(x, w, csr), "D1": lambda: PF.conv_forward_d1(x, w, km)}
        res = {name: _timed(fn, flush, iters, warmup) for name, fn in fns.items() if both or name == pick}
        row = _conv_row(f"indoor subm3 {c}x{c}", res[pick], km.n_in, km.n_in, pairs, 27, c, c, 2, pk)
        row.update({"C": c, "auto": pick})
        if both:
            row.update({"D2_us": res["D2"] * 1e6, "D1_us": res["D1"] * 1e6,
                        "auto_is_faster": res[pick] <= min(res.values()) * 1.02})
        rows.append(row)
    return rows, dict(voxels=km.n_in, surface_samples=samples, pairs=pairs, pairs_per_voxel=pairs / km.n_in)


def selector_rows(dev, iters: int = 5, warmup: int = 2):
    """``--workload selector``: both dataflows on clouds that span the selector's inputs -- channel width
    (16..256), sparsity (indoor surfaces ~2.7 pairs per row, LiDAR ~3.4, a fully dense block 27) and map
    size (about 25 k and 200 k rows) -- submanifold 3x3x3, fp16, kernel-only, L2 flushed.  The table
    ``pcengine_b200.spconv._D1_WINS`` is what this sweep says."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    synth = _synth()

    def lidar(n_target):
        if n_target > 100000:
            return np.concatenate([synth.with_batch(synth.lidar_scan(2000 + i), i) for i in range(3)])
        xyz = synth.lidar_scan(2000)
        centre = np.median(xyz, axis=0)
        d = np.abs(xyz - centre).max(axis=1)
        return synth.with_batch(xyz[d <= np.sort(d)[min(n_target, len(d)) - 1]])

    def block(side):
        g = np.arange(side)
        xyz = np.stack(np.meshgrid(g, g, g, indexing="ij"), -1).reshape(-1, 3)
        return synth.with_batch(xyz.astype(np.int32))

    clouds = [("indoor", 25000, lambda: synth.with_batch(synth.indoor_room(3001, 25000)[0])),
              ("indoor", 200000, lambda: synth.with_batch(synth.indoor_room(3001, 200000)[0])),
              ("lidar", 25000, lambda: lidar(25000)), ("lidar", 200000, lambda: lidar(200000)),
              ("dense", 24389, lambda: block(29)), ("dense", 195112, lambda: block(58))]
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    rows = []
    g = torch.Generator().manual_seed(3)
    for name, _, make in clouds:
        coords_h = make()
        coords = torch.from_numpy(np.ascontiguousarray(coords_h)).to(dev)
        km = pce.KernelMap(coords, (3, 3, 3), (1, 1, 1), (0, 0, 0), [0, 0, 0], coords_h[:, 1:].max(0).tolist(), True)
        csr = km.csr()
        pairs = int(csr.rowptr[-1].item())
        for c in (16, 32, 64, 96, 128, 256):
            x = torch.randn(km.n_in, c, generator=g).half().to(dev)
            w = (torch.randn(27, c, c, generator=g) / (27 * c) ** 0.5).half().to(dev)
            t2 = _timed(lambda: PF.conv_forward(x, w, csr), flush, iters, warmup)
            t1 = _timed(lambda: PF.conv_forward_d1(x, w, km), flush, iters, warmup)
            rows.append({"cloud": name, "rows": km.n_in, "pairs_per_row": round(pairs / km.n_in, 2), "C": c,
                         "D2_us": round(t2 * 1e6, 1), "D1_us": round(t1 * 1e6, 1), "D1_over_D2": round(t1 / t2, 2)})
            del x, w
        del km, csr
        torch.cuda.empty_cache()
    return rows


def scene_rows(dev, pk, rank: int, world: int, cases, steps: int, warmup: int):
    """ONE large indoor scene (20 rooms tiled 5x4, about 1.5 M voxels at 2 cm) split into x-slabs, one per
    rank, with a kernel-radius halo.  Per layer shape of ``cases`` ((kernel size, channels), ...): time per
    layer of a stack of 8 layers queued back to back, the halo exchange of every layer inside the timed
    region, kernel-map construction outside it; max over ranks."""
    import torch.distributed as dist

    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    from pcengine_b200 import multigpu as mg
    synth = _synth()
    xyz = synth.tiled_scene()
    coords_h = synth.with_batch(xyz)
    cmax = coords_h[:, 1:].max(0).tolist()
    n_total = len(coords_h)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    rows = []
    STACK = 8  # layers queued back to back per timing
    for ks, c in cases:
        radius = (ks - 1) // 2
        cuts, owned = mg.split_scene(coords_h, world, radius)
        idx = owned[rank]
        scene = mg.SlabScene(torch.from_numpy(coords_h[idx]).to(dev), cuts, rank, world, radius).setup()
        g = torch.Generator().manual_seed(11 + rank)
        feats = scene.alloc_local(c, torch.float16)
        feats[: scene.n_owned] = torch.randn(len(idx), c, generator=g).half().to(dev)
        w = (torch.randn(ks ** 3, c, c, generator=torch.Generator().manual_seed(3)) / (ks ** 3 * c) ** 0.5).half().to(dev)
        km = pce.KernelMap(scene.local_coords, (ks,) * 3, (1, 1, 1), (0, 0, 0), [0, 0, 0], cmax, True)
        csr = km.csr().restrict(scene.n_owned)  # this rank computes its owned rows, not the halo's
        pairs = int(csr.rowptr[scene.n_owned].item())  # pairs whose output this rank owns
        push, exchange = None, "none (one slab)"
        if world > 1:
            try:  # boundary rows stored into the neighbours' halos by the convolution's own epilogue
                push = mg.PeerPush(scene, c, torch.float16)
                push.local(0).copy_(feats)
                scene.exchange_into(push.local(0))
                exchange = "peer stores from the convolution epilogue + one symmetric-memory barrier per layer"
            except Exception as e:  # no symmetric memory on this system: messages before the layer
                push, exchange = None, f"NCCL isend/irecv before the layer (peer push unavailable: {type(e).__name__})"

        def layer(i: int):
            if push is None:
                return PF.conv_forward(scene.exchange_into(feats), w, csr)
            src, dst = i & 1, (i & 1) ^ 1
            out = PF.conv_forward(push.local(src), w, csr, push.epilogue(dst), out=push.owned(dst))
            push.barrier(dst)
            return out

        it = 0
        for _ in range(max(warmup, 2)):
            layer(it)
            it += 1
        ts = []
        for _ in range(max(steps, 3)):
            flush.zero_()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(STACK):  # a stack of layers, so that launch latency on an idle GPU is not what is timed
                out = layer(it)
                it += 1
            b.record()
            b.synchronize()
            ts.append(mg.max_over_ranks(a.elapsed_time(b) * 1e-3, dev) / STACK)
        t = float(np.median(ts))
        tot_pairs = pairs
        halo_rows = int(scene.local_coords.size(0) - scene.n_owned)
        if world > 1:
            tp = torch.tensor([pairs, halo_rows], dtype=torch.int64, device=dev)
            dist.all_reduce(tp)
            tot_pairs, halo_rows = int(tp[0]), int(tp[1])
        by = 2 * (n_total * c * 2) + 2 * ks ** 3 * c * c + 4 * tot_pairs
        fl = 2.0 * tot_pairs * c * c
        rows.append({"layer": f"subm{ks}_{c}x{c}", "ms": t * 1e3, "voxels_per_s": n_total / t, "pairs": tot_pairs,
                     "halo_rows_total": halo_rows, "exchange": exchange, "GB/s": by / t / 1e9, "TFLOP/s": fl / t / 1e12,
                     "hbm_frac_per_gpu": by / t / 1e9 / pk["hbm_gbs"] / world, "tensor_frac_per_gpu": fl / t / 1e12 / pk["tflops"] / world})
        del km, csr, scene, feats, w, out, push
        torch.cuda.empty_cache()
    return {"workload": "scene_slabs", "n_gpus": world, "voxels": n_total, "layers": rows,
            "note": "x-slabs; time per layer of a stack of 8 layers queued back to back, the kernel-radius "
                    "halo exchange of every layer inside the timed region, map build outside it"}


def run_scene(args):
    """``--workload scene``: every layer shape of the large-scene configuration (3^3 and 5^3, C = 64 and 256)."""
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    res = scene_rows(dev, peaks(), rank, world, ((3, 64), (3, 256), (5, 64), (5, 256)), args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.destroy_process_group()


def run_scene_unet(args):
    """``--workload scene_unet``: the MinkUNet over the ONE large indoor scene (about 1.5 M voxels), the scene
    cut into x-slabs at multiples of 16 voxels, one slab per rank (``spTensor.slabs``): every submanifold layer
    exchanges its level's halo rows, the 2x2x2 layers exchange nothing.  Forward passes per second (kernel maps
    kept: the scene is static), max over ranks; at one rank also the ordinary pass on the undivided tensor and
    the largest difference between the two."""
    import torch.distributed as dist

    import pcengine_b200 as pce
    from pcengine_b200 import multigpu as mg
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    synth = _synth()
    coords_h = synth.with_batch(synth.tiled_scene())
    cmax = coords_h[:, 1:].max(0).tolist()
    model = pce.MinkUNet(IN_CHANNELS, NUM_CLASSES)
    model.load_state_dict(seeded_state_dict({k: tuple(v.shape) for k, v in model.state_dict().items()}))
    model = model.half().eval().to(dev)
    feats_h = torch.randn(len(coords_h), IN_CHANNELS, generator=torch.Generator().manual_seed(21)).half()
    cuts, owned = mg.split_scene(coords_h, world, 1, align=16)
    idx = owned[rank]
    coords = torch.from_numpy(coords_h[idx]).to(dev)
    feats = feats_h[idx].to(dev)
    levels = mg.SlabLevels(coords, cuts, rank, world, 1, [2, 2, 2, 2], cmax)
    kept = {}

    def forward(slabs):
        x = pce.spTensor(feats, coords, None, [0, 0, 0], cmax, init_tag=pce.MinkUNet.tags())
        x.slabs = slabs
        x.kmaps = kept.setdefault(id(slabs), {})  # a static scene: the maps of the first pass serve the later ones
        if x.kmaps:
            x.init_tag = ["auto"]
        with torch.no_grad():
            return model(x).feats

    def timed(slabs):
        for _ in range(max(args.warmup, 2)):
            forward(slabs)
        ts = []
        for _ in range(max(args.steps, 5)):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = forward(slabs)
            b.record()
            b.synchronize()
            ts.append(mg.max_over_ranks(a.elapsed_time(b) * 1e-3, dev))
        return float(np.median(ts)), out
    t_slab, y_slab = timed(levels)
    halo = sum(int(sc.n_local - sc.n_owned) for sc in levels.scenes)
    if world > 1:
        h = torch.tensor([halo], dtype=torch.int64, device=dev)
        dist.all_reduce(h)
        halo = int(h)
    res = {"workload": "scene_unet", "n_gpus": world, "voxels": len(coords_h), "cuts": cuts, "ms_per_pass": t_slab * 1e3,
           "voxels_per_s": len(coords_h) / t_slab, "halo_rows_all_levels": halo,
           "exchange": "none (one slab)"}
    if world > 1:
        boxed = [k for k, v in levels.__dict__.get("_mailboxes", {}).items() if v is not None]
        res["exchange"] = ("boundary rows stored into the neighbours' mailboxes (peer stores) + one symmetric-memory "
                           f"barrier per submanifold layer ({len(boxed)} level/width pairs; NCCL messages for the rest)"
                           if boxed else "NCCL isend/irecv of the halo rows before every submanifold layer")
    model.plan_ahead = False  # the ordinary per-layer pass on the undivided tensor, maps kept as well
    if world == 1:
        t_whole, y_whole = timed(None)
        res["ms_per_pass_without_slabs"] = t_whole * 1e3
        res["max_abs_diff"] = float((y_slab.float() - y_whole.float()).abs().max())
    else:  # every rank also runs the undivided scene once and compares the rows it owns
        with torch.no_grad():
            whole = model(pce.spTensor(feats_h.to(dev), torch.from_numpy(coords_h).to(dev), None, [0, 0, 0], cmax,
                                       init_tag=pce.MinkUNet.tags())).feats
        want = whole[torch.from_numpy(idx).to(dev)].float()
        err = (y_slab.float() - want).norm() / want.norm().clamp_min(1e-20)
        res["rel_l2_vs_undivided_max_over_ranks"] = mg.max_over_ranks(float(err), dev)
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.destroy_process_group()


def run_indoor(args):
    """``--workload indoor``: the indoor-room sweep with both dataflows."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    rows, info = indoor_rows(dev, peaks(), max(args.steps, 5), max(args.warmup, 2), both=True)
    print(json.dumps({"workload": "indoor_sweep", **info, "layers": rows}))


def run_selector(args):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    print(json.dumps({"workload": "selector_sweep", "rows": selector_rows(dev, max(args.steps, 5), max(args.warmup, 2))}))


def run_layer(args):
    """``--layer NAME``: only that single layer on ``--scans`` collated scans (a small, short case for
    a profiler capture).  Prints one JSON line with the kernel-only figures."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    rows, n = layer_table(dev, peaks(), [args.layer], scans=args.scans, iters=args.steps, warmup=args.warmup,
                          level=args.level)
    print(json.dumps({"workload": "single_layer", "voxels": n, "scans": args.scans, "level": args.level, **rows[0]}))


def _host_array(a) -> np.ndarray:
    t = a.tensor() if hasattr(a, "tensor") else a
    return t.detach().cpu().numpy()


def check_parity(model_maps: dict, gpu_logits: torch.Tensor, oracle_logits: torch.Tensor, oracle_maps: dict) -> dict:
    """Kernel maps of the timed batch against the oracle's, bit for bit (indicator map, kpos, qkpos,
    output coordinates of every map the pass built), and the logits' rel-L2."""
    from oracle import conv_oracle as co
    from oracle import kmap_oracle as ko
    ones = ko.encode3((1, 1, 1))
    checked, exact = 0, True
    for (ks_code, tstride_code, stride_code), km in model_maps.items():
        level = int(round(np.log2(ko.decode3(tstride_code)[0])))
        want = oracle_maps.get(("subm" if stride_code == ones else "down", level))
        if want is None:
            exact = False
            continue
        checked += 1
        for name in ("map", "kpos", "qkpos", "out_coords"):
            if not np.array_equal(_host_array(getattr(km, name)).reshape(-1), np.asarray(want[name]).reshape(-1)):
                exact = False
    exact = exact and checked == len(oracle_maps)
    err = co.rel_l2(gpu_logits.float().cpu(), oracle_logits.float())
    return {"maps_bit_exact": bool(exact), "maps_checked": checked, "logits_rel_l2": err, "tol": PARITY_TOL,
            "ok": bool(exact and err <= PARITY_TOL)}


class _Batch:
    """One rank's collated scans: pinned host copies, device-resident copies, and the loops timed on them."""

    def __init__(self, ids, model, dev, flush):
        import pcengine_b200 as pce
        self.pce, self.model, self.dev, self.flush, self.ids = pce, model, dev, flush, list(ids)
        self.coords_h, feats_h, self.sizes = make_scans(ids)
        self.cmax = self.coords_h[:, 1:].max(0).tolist()
        self.coords_pin = torch.from_numpy(self.coords_h).pin_memory()
        self.feats_pin = feats_h.pin_memory()
        self.coords_d = self.coords_pin.to(dev)
        self.feats_d = self.feats_pin.to(dev)
        self.resident = torch.cuda.Event()  # the device-resident inputs exist from here on
        self.resident.record()

    def tensor(self, c, f, ready=None):
        x = self.pce.spTensor(f, c, None, [0, 0, 0], self.cmax, batchsize=len(self.ids), init_tag=self.pce.MinkUNet.tags())
        x.coords_ready = ready  # lets the map planner start as soon as the coordinates exist
        return x

    def forward_once(self):
        with torch.no_grad():
            return self.model(self.tensor(self.coords_d, self.feats_d, self.resident))

    def steps_planned_one_ahead(self, n: int):
        """n forward passes, each preceded by the start of the NEXT pass's map construction
        (model.plan): every step holds one map construction and one forward pass, and the maps of a
        batch are being built while the batch before it computes.  The pass planned last is dropped."""
        nxt = self.tensor(self.coords_d, self.feats_d, self.resident)
        self.model.plan(nxt)
        for _ in range(n):
            self.flush.zero_()
            cur, nxt = nxt, self.tensor(self.coords_d, self.feats_d, self.resident)
            self.model.plan(nxt)
            with torch.no_grad():
                self.model(cur)

    def make_server(self):
        """End to end: pinned host -> device, forward, logits -> pinned host.  A serving loop with two
        batches in flight: batch i's inputs are copied on an input stream (the map planner starts on
        their arrival), its logits leave on an output stream, and the host waits for batch i-1's logits
        once batch i is queued.  Every step moves its own inputs and its own result; buffers are double."""
        dev, model = self.dev, self.model
        main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        c_buf = [torch.empty_like(self.coords_d) for _ in range(2)]
        f_buf = [torch.empty_like(self.feats_d) for _ in range(2)]
        l_pin = [torch.empty((len(self.coords_h), NUM_CLASSES), dtype=torch.float16).pin_memory() for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]     # inputs of the batch are on the device
        ev_done = [torch.cuda.Event() for _ in range(2)]   # the batch is computed (its input buffers are free)
        ev_out = [torch.cuda.Event() for _ in range(2)]    # its logits are on the host
        outs = [None, None]                                # device logits, alive until their copy was waited for
        self.h2d_bytes = int(self.coords_pin.numel() * 4 + self.feats_pin.numel() * 2)
        self.d2h_bytes = int(l_pin[0].numel() * 2)

        def upload(i: int):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_done[b])
                c_buf[b].copy_(self.coords_pin, non_blocking=True)
                f_buf[b].copy_(self.feats_pin, non_blocking=True)
                ev_in[b].record(s_in)
            x = self.tensor(c_buf[b], f_buf[b], ev_in[b])
            model.plan(x)
            return x

        def serve(n_batches: int):
            nxt = upload(0)
            for i in range(n_batches):
                b = i & 1
                cur = nxt
                if i + 1 < n_batches:
                    nxt = upload(i + 1)  # the next batch's copy and maps overlap this batch's forward pass
                main.wait_event(ev_in[b])
                self.flush.zero_()
                with torch.no_grad():
                    outs[b] = model(cur).feats
                ev_done[b].record(main)
                s_out.wait_event(ev_done[b])
                with torch.cuda.stream(s_out):
                    l_pin[b].copy_(outs[b], non_blocking=True)
                    ev_out[b].record(s_out)
                if i >= 1:
                    ev_out[b ^ 1].synchronize()
            ev_out[(n_batches - 1) & 1].synchronize()

        return serve


def run_ours(args):
    import torch.distributed as dist

    import pcengine_b200 as pce
    from pcengine_b200 import _lib
    from pcengine_b200 import functional as PF

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    all_cores = sorted(os.sched_getaffinity(0))
    host_cores = len(all_cores)
    if world > 1 and args.pin:
        # one share of the host cores per rank: the rank's main thread and the planner's threads stay
        # off the other ranks' cores
        share = host_cores // world
        if share >= 4:  # a rank keeps four threads busy (its main thread and the planner's three)
            os.sched_setaffinity(0, all_cores[local * share:(local + 1) * share])
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    per_rank = {}

    def max_over_ranks(x: float, name: str, steps: int) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        every = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        per_rank[name] = [round(float(v.item()) / steps * 1e3, 3) for v in every]
        return max(float(v.item()) for v in every)

    pk = peaks()
    model = pce.MinkUNet(IN_CHANNELS, NUM_CLASSES)
    model.load_state_dict(seeded_state_dict({k: tuple(v.shape) for k, v in model.state_dict().items()}))
    model = model.half().eval().to(dev)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    steps, warmup = max(1, args.steps), max(args.warmup, 3)

    def device_timed(batch: "_Batch", name: str):
        """W warm-up steps, then K steps between barrier + synchronize on both sides; max over ranks."""
        for _ in range(2):  # set-up, not warm-up: packs the weights, lets the planner create its storage
            batch.forward_once()
            torch.cuda.synchronize()
        batch.steps_planned_one_ahead(warmup)
        launches0 = _lib.lib.pce_kernel_launches()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        batch.steps_planned_one_ahead(steps)
        e1.record()
        barrier()
        dt = max_over_ranks(e0.elapsed_time(e1) * 1e-3, name, steps)
        return dt, int(_lib.lib.pce_kernel_launches() - launches0)

    # ---- the batch of 8 scans, sharded over the ranks ----------------------------------------
    my_ids = scans_for_rank(BATCH_SCANS, rank, world)
    if not my_ids:
        raise SystemExit(f"{world} ranks for a batch of {BATCH_SCANS} scans: at most {BATCH_SCANS} GPUs")
    batch = _Batch(my_ids, model, dev, flush)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dt, launches = device_timed(batch, "ms_per_step")
    # ---- the same K steps again with a CUDA-event pair around every convolution launch ------
    # (kept out of the loop above: ~80 extra event records per step perturb the headline time)
    PF.PROFILE = []
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    batch.steps_planned_one_ahead(steps)
    p1.record()
    barrier()
    dt_prof = p0.elapsed_time(p1) * 1e-3
    prof, PF.PROFILE = PF.PROFILE, None
    # ---- end to end ---------------------------------------------------------------------------
    serve = batch.make_server()
    serve(warmup)  # warm-up of this loop's own streams and allocation pattern
    barrier()
    t0 = time.perf_counter()
    serve(steps)
    dt_e2e = max_over_ranks(time.perf_counter() - t0, "e2e_ms_per_step", steps)
    clocks = sampler.stop() if rank == 0 else None
    # ---- weak-scaling side figure: 8 scans of its own on every rank ----------------------------
    weak = None
    if world > 1 and not args.lean:
        wb = _Batch([SCANS_PER_GPU * rank + i for i in range(SCANS_PER_GPU)], model, dev, flush)
        dt_w, _ = device_timed(wb, "weak_ms_per_step")
        weak = SCANS_PER_GPU * world * steps / dt_w
        del wb
    # ---- roofline of the dominant convolution kernel ---------------------------------------
    by_kernel = {}
    by_shape = {}
    t_min_convs = 0.0
    for rec in prof:
        t = rec["start"].elapsed_time(rec["end"]) * 1e-3
        pairs = int(rec["pairs"].item())
        e = rec["esize"]
        byt = e * (rec["n_in"] * rec["cin"] + rec["n_out"] * rec["cout"]) + e * rec["kv"] * rec["cin"] * rec["cout"] + 4 * pairs
        flops = 2.0 * pairs * rec["cin"] * rec["cout"]
        if rec["extra_c"]:  # second operand: its rows and weights are read, one more product per row
            byt += e * rec["extra_c"] * (rec["n_out"] + rec["cout"])
            flops += 2.0 * rec["n_out"] * rec["extra_c"] * rec["cout"]
        if rec["residual"]:
            byt += e * rec["n_out"] * rec["cout"]
        t_min_convs += max(byt / (pk["hbm_gbs"] * 1e9), flops / (pk["tflops"] * 1e12))
        k = by_kernel.setdefault(rec["kernel"], dict(t=0.0, bytes=0.0, flops=0.0, n=0))
        k["t"] += t
        k["bytes"] += byt
        k["flops"] += flops
        k["n"] += 1
        sh = by_shape.setdefault((rec["kernel"], rec["n_out"], rec["kv"], rec["cin"], rec["cout"]), [0, 0.0, 0.0, 0.0])
        sh[0] += 1
        sh[1] += t
        sh[2] += byt
        sh[3] += flops
    # Lower bound of a step: every convolution at the better of its two roofs plus every kernel map at
    # the copy bandwidth over its algorithmic bytes (coordinates in, table payload, 12 B per lookup,
    # neighbour table out, output coordinates of a strided map).
    t_min = t_min_convs / steps
    last = batch.forward_once()
    gpu_logits, maps = last.feats, last.kmaps
    for km in maps.values():
        lookups = km.n_out * (km.kv - (1 if km.subm else 0))
        map_bytes = 28 * km.n_in + 12 * lookups + 4 * km.n_out * km.kv + (0 if km.subm else 16 * km.n_out)
        t_min += map_bytes / (pk["hbm_gbs"] * 1e9)
    roof = None
    if by_kernel:
        name, k = max(by_kernel.items(), key=lambda kv: kv[1]["t"])
        ach = k["bytes"] / k["t"] / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                "traffic": None, "kernel": name, "launches_timed": k["n"], "avg_launch_us": k["t"] / k["n"] * 1e6,
                "share_of_step": k["t"] / (dt_prof if dt_prof > 0 else 1.0),
                "timed_loop_ms_per_step": dt_prof / steps * 1e3,
                "tensor_tflops": k["flops"] / k["t"] / 1e12, "tensor_frac": k["flops"] / k["t"] / 1e12 / pk["tflops"],
                "peak_source": pk["source"], "note": "sum of algorithmic bytes of every launch of this kernel in the "
                "K steps run right after the timed ones / sum of their CUDA-event durations; traffic is null "
                "because the aggregate spans every launch shape of a step (DRAM bytes of single shapes: profiles/). The "
                "event pairs sit around per-layer launches (timed_loop_ms_per_step is that loop's own step): where "
                "the host, not the GPU, paces that loop (a scan or two per rank) a pair also holds launch latency, "
                "and the launches of a step can sum to more than the one-call step the headline times"}
    # ---- extras ------------------------------------------------------------------------------
    layers = cpu = parity = config1 = indoor = scene = None
    cores_per_rank = len(os.sched_getaffinity(0))
    if not args.lean:
        scene = scene_rows(dev, pk, rank, world, ((3, 64), (3, 256)), 3, 2)  # every rank takes part
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    if not args.lean and world == 1:
        layers, _ = layer_table(dev, pk, with_reference=True)
        config1 = config1_row(dev, pk)
        indoor, indoor_info = indoor_rows(dev, pk, both=False)
        indoor = {**indoor_info, "layers": indoor}
        os.sched_setaffinity(0, all_cores)
        cpu_v, cpu_dt, cores, sample, o_logits, o_maps = oracle_pass(my_ids, 1, 0, want_outputs=True)
        cpu = {"value": cpu_v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        parity = check_parity(maps, gpu_logits, o_logits, o_maps)
    elif not args.lean:
        # N > 1: the other ranks have left; rank 0 checks ITS shard of the batch against the oracle on all
        # host cores (the CPU baseline itself is the N = 1 line's and the reference arm's)
        dist.destroy_process_group()
        cores_per_rank = len(os.sched_getaffinity(0))
        os.sched_setaffinity(0, all_cores)
        _, _, _, _, o_logits, o_maps = oracle_pass(my_ids, 1, 0, want_outputs=True)
        parity = check_parity(maps, gpu_logits, o_logits, o_maps)
        parity["scans_checked"] = list(my_ids)
    del maps, last
    total_scans = BATCH_SCANS * steps
    value = total_scans / dt
    if parity is not None and not parity["ok"]:
        value = None  # a fast result that differs from the oracle's is not a result
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "minkunet_lidar_batch8", "batch_scans": BATCH_SCANS, "scans_per_gpu": len(my_ids),
                   "voxels_rank0": int(len(batch.coords_h)), "voxels_per_scan_rank0": batch.sizes,
                   "in_channels": IN_CHANNELS, "classes": NUM_CLASSES,
                   "widths": "32-32-64-128-256-256-128-96-96", "map_build": "inside the timed step (planner threads, own streams), started one batch ahead (model.plan)",
                   "e2e_loop": "two batches in flight: H2D on an input stream and the batch's map construction start while the batch before it computes, D2H on an output stream, host waits for the previous batch's logits",
                   "l2": "192 MiB memset between steps, inside the timed region", "accumulate": "fp32"},
        "e2e": {"value": total_scans / dt_e2e, "unit": UNIT,
                "h2d_bytes_per_step": batch.h2d_bytes, "d2h_bytes_per_step": batch.d2h_bytes,
                "ms_per_step": dt_e2e / steps * 1e3},
        "gpu_launches": launches,
        "parity": parity,
        "roofline": roof,
        "network_roofline": {"t_min_ms": t_min * 1e3, "t_measured_ms": dt / steps * 1e3,
                             "frac": t_min / (dt / steps),
                             "note": "rank 0's share: sum over the step's convolutions of max(bytes/copy bandwidth, "
                                     "flops/GEMM peak) plus its kernel maps' algorithmic bytes / copy bandwidth, over the measured step"},
        "kernels": {k: {"launches": v["n"], "ms": v["t"] * 1e3} for k, v in by_kernel.items()},
        "conv_shapes": [{"kernel": k[0], "n_out": k[1], "kv": k[2], "cin": k[3], "cout": k[4], "launches": v[0],
                         "us_per_launch": v[1] / v[0] * 1e6, "GB/s": v[2] / v[1] / 1e9, "TFLOP/s": v[3] / v[1] / 1e12}
                        for k, v in sorted(by_shape.items(), key=lambda kv: -kv[1][1])][:16],
        "layers": layers,
        "config1": config1,
        "indoor_sweep": indoor,
        "scene_slabs": scene,
        "cpu_baseline": cpu,
        "clocks": clocks,
    }
    if world > 1:
        line["weak_scans_per_s"] = weak
        line["per_rank"] = {**per_rank, "host_cores": host_cores, "cores_per_rank": cores_per_rank,
                            "pinned": bool(args.pin)}
    print(json.dumps(line))
    if world > 1 and dist.is_initialized():
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    ap.add_argument("--layer", type=str, default=None, choices=sorted(LAYERS),
                    help="run one single layer only (kernel-only timing); see --scans")
    ap.add_argument("--scans", type=int, default=8, help="collated scans for --layer")
    ap.add_argument("--level", type=int, default=0, choices=range(5),
                    help="--layer: run on the coordinates after this many 2x2x2 / stride-2 down-samplings")
    ap.add_argument("--workload", type=str, default="minkunet", choices=["minkunet", "scene", "scene_unet", "indoor", "selector"],
                    help="minkunet: the batch of 8 LiDAR scans (default); scene: one 1.5 M-voxel scene in x-slabs, single layers; "
                         "scene_unet: the MinkUNet over that scene on slabs; indoor: the room sweep, both dataflows")
    ap.add_argument("--no-pin", dest="pin", action="store_false",
                    help="multi-rank runs: do not give each rank its own share of the host cores")
    ap.add_argument("--lean", action="store_true",
                    help="skip the per-layer tables, the scene, the parity check and the CPU baseline (short runs under a profiler)")
    args = ap.parse_args()
    if args.workload == "scene_unet":
        return run_scene_unet(args)
    if args.workload == "scene":
        run_scene(args)
    elif args.workload == "indoor":
        run_indoor(args)
    elif args.workload == "selector":
        run_selector(args)
    elif args.layer is not None:
        run_layer(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
