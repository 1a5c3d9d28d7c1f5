"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched through torchrun)
    python bench.py --impl reference --gpus N --steps K --warmup W

Workload (``config.workload`` = "minkunet_lidar_batch8"): one step is one inference pass of the
MinkUNet-shaped network (fp16, random-init, seed 4001) over a collated batch of 8 synthetic
64-beam LiDAR scans per GPU (seeds 2000 + 8*rank + i), kernel-map construction included.
Every rank works on its own scans and no collective touches the data path (weak scaling).

The single JSON line carries: the device-timed whole-job throughput with inputs resident in HBM
(``value``), the same metric through host buffers with the copies inside the timed region
(``e2e``), the roofline of the dominant convolution kernel from per-launch CUDA events recorded
inside the timed steps, per-layer figures for the single LiDAR layers (``layers``), the CPU
oracle timed on the host cores (``cpu_baseline``) and the GPU clocks sampled during the run.
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

SCANS_PER_GPU = 8
IN_CHANNELS = 4
NUM_CLASSES = 19
WEIGHT_SEED = 4001
METRIC = "minkunet_scans_per_s"
UNIT = "scans/s"


# ----------------------------------------------------------------------------- inputs
def make_batch(rank: int, n_scans: int = SCANS_PER_GPU):
    """Collated int32 coords [N,4] and fp16 features [N,4] of this rank's scans (host, NumPy/torch)."""
    from pcengine_b200 import synth
    coords, sizes = [], []
    for i in range(n_scans):
        xyz = synth.lidar_scan(2000 + SCANS_PER_GPU * rank + i)
        coords.append(synth.with_batch(xyz, i))
        sizes.append(len(xyz))
    coords = np.concatenate(coords)
    g = torch.Generator().manual_seed(9000 + rank)
    feats = torch.randn(len(coords), IN_CHANNELS, generator=g).half()
    return coords, feats, sizes


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
def oracle_scans_per_s(rank: int, steps: int, warmup: int, n_scans: int = SCANS_PER_GPU):
    """The CPU restatement (oracle) on ``n_scans`` of this rank's scans per step."""
    import pcengine_b200 as pce
    from oracle import minkunet_oracle as mo
    torch.set_num_threads(os.cpu_count() or 1)
    coords, feats, sizes = make_batch(rank, n_scans)
    torch.manual_seed(WEIGHT_SEED)
    model = pce.MinkUNet(IN_CHANNELS, NUM_CLASSES)
    pce.randomize_batchnorm(model, WEIGHT_SEED)
    sd = model.half().eval().state_dict()
    for _ in range(warmup):
        mo.forward(sd, coords, feats)
    t0 = time.perf_counter()
    for _ in range(steps):
        mo.forward(sd, coords, feats)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return n_scans / dt, dt, torch.get_num_threads(), f"{n_scans} scan(s) of the batch ({sum(sizes)} voxels) per step"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    v, dt, cores, sample = oracle_scans_per_s(0, max(1, min(args.steps, 3)), min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "minkunet_lidar_batch8", "note": "CPU oracle (NumPy maps + PyTorch CPU gather-matmul-scatter, "
                   "fp32 arithmetic on fp16 values); the reference has no CPU implementation and its CUDA build is not "
                   "run here", "sample": sample, "timed_steps": max(1, min(args.steps, 3))},
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


def layer_table(dev, pk, names=None, scans: int = 1, iters: int = 10, warmup: int = 3):
    """Single LiDAR-shaped layers on ``scans`` collated scans (seeds 2000..): kernel-only time per layer
    with an L2 flush between launches; algorithmic bytes / flops per launch against the measured peaks."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    coords_h, _, _ = make_batch(0, scans)
    coords = torch.from_numpy(coords_h).to(dev)
    cmax = coords_h[:, 1:].max(0).tolist()
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    names = list(names or DEFAULT_LAYERS)
    maps = {}

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
        for _ in range(warmup):
            PF.conv_forward(x, w, csr)
        ts = []
        for _ in range(iters):
            _host_lead()
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            PF.conv_forward(x, w, csr)
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3)
        t = float(np.median(ts))
        by = 2 * (csr.n_src * cin + csr.n_rows * cout) + 2 * kv * cin * cout + 4 * pairs
        fl = 2.0 * pairs * cin * cout
        rows.append({"layer": name, "n_in": csr.n_src, "n_out": csr.n_rows, "pairs": pairs, "us": t * 1e6,
                     "GB/s": by / t / 1e9, "TFLOP/s": fl / t / 1e12, "hbm_frac": by / t / 1e9 / pk["hbm_gbs"],
                     "tensor_frac": fl / t / 1e12 / pk["tflops"], "alg_bytes": by, "alg_flops": fl})
    return rows, int(coords.size(0))


def run_scene(args):
    """``--workload scene``: ONE large indoor scene (20 rooms tiled 5x4, about 1.5 M voxels at 2 cm)
    split into x-slabs, one per rank, with a kernel-radius halo exchanged by point-to-point messages
    (NCCL over NVLink) before every layer.  Per layer: time of [halo exchange + convolution] over all
    ranks (max), voxels/s of the whole scene, algorithmic GB/s and TFLOP/s."""
    import torch.distributed as dist

    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    from pcengine_b200 import multigpu as mg
    from pcengine_b200 import synth
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pk = peaks()
    xyz = synth.tiled_scene()
    coords_h = synth.with_batch(xyz)
    cmax = coords_h[:, 1:].max(0).tolist()
    n_total = len(coords_h)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    rows = []
    STACK = 8  # layers queued back to back per timing
    for ks, c in ((3, 64), (3, 256), (5, 64), (5, 256)):
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
            except Exception as e:  # no symmetric memory on this system: messages after the layer
                push, exchange = None, f"NCCL isend/irecv before the layer (peer push unavailable: {type(e).__name__})"

        def layer(i: int):
            if push is None:
                return PF.conv_forward(scene.exchange_into(feats), w, csr)
            src, dst = i & 1, (i & 1) ^ 1
            out = PF.conv_forward(push.local(src), w, csr, push.epilogue(dst), out=push.owned(dst))
            push.barrier(dst)
            return out

        it = 0
        for _ in range(max(args.warmup, 2)):
            layer(it)
            it += 1
        ts = []
        for _ in range(max(args.steps, 3)):
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
    if rank == 0:
        print(json.dumps({"workload": "scene_slabs", "n_gpus": world, "voxels": n_total, "layers": rows,
                          "note": "x-slabs; time per layer of a stack of 8 layers queued back to back, the kernel-radius "
                                  "halo exchange of every layer inside the timed region, map build outside it"}))
    if world > 1:
        dist.destroy_process_group()


def run_indoor(args):
    """``--workload indoor``: the indoor-room sweep.  One 8x8x3 m room voxelised at 2 cm (about 200 k
    voxels), submanifold 3x3x3 at C_in = C_out in {16, 32, 64, 96, 128, 256}, fp16: the fused
    output-stationary dataflow (D2) and the explicit gather -> GEMM -> scatter dataflow (D1), kernel-only
    with an L2 flush between launches, plus what the 'auto' selector picks."""
    import pcengine_b200 as pce
    from pcengine_b200 import functional as PF
    from pcengine_b200 import synth
    from pcengine_b200.spconv import _choose_dataflow
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    pk = peaks()
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
        res = {}
        for name, fn in (("D2", lambda: PF.conv_forward(x, w, csr)), ("D1", lambda: PF.conv_forward_d1(x, w, km))):
            for _ in range(max(args.warmup, 2)):
                fn()
            ts = []
            for _ in range(max(args.steps, 5)):
                _host_lead()
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                b.synchronize()
                ts.append(a.elapsed_time(b) * 1e-3)
            res[name] = float(np.median(ts))
        by = 2 * (2 * km.n_in * c) + 2 * 27 * c * c + 4 * pairs
        fl = 2.0 * pairs * c * c
        pick = _choose_dataflow("auto", c, c)
        rows.append({"C": c, "D2_us": res["D2"] * 1e6, "D1_us": res["D1"] * 1e6, "auto": pick,
                     "auto_is_faster": res[pick] <= min(res.values()) * 1.02,
                     "GB/s": by / res[pick] / 1e9, "TFLOP/s": fl / res[pick] / 1e12,
                     "hbm_frac": by / res[pick] / 1e9 / pk["hbm_gbs"], "tensor_frac": fl / res[pick] / 1e12 / pk["tflops"]})
    print(json.dumps({"workload": "indoor_sweep", "voxels": km.n_in, "surface_samples": samples, "pairs": pairs,
                      "pairs_per_voxel": pairs / km.n_in, "layers": rows}))


def run_layer(args):
    """``--layer NAME``: only that single layer on ``--scans`` collated scans (a small, short case for
    a profiler capture).  Prints one JSON line with the kernel-only figures."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    rows, n = layer_table(dev, peaks(), [args.layer], scans=args.scans, iters=args.steps, warmup=args.warmup)
    print(json.dumps({"workload": "single_layer", "voxels": n, "scans": args.scans, **rows[0]}))


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
    host_cores = len(os.sched_getaffinity(0))
    if world > 1 and args.pin:
        # one share of the host cores per rank: the rank's main thread and the planner's threads stay
        # off the other ranks' cores
        cores = sorted(os.sched_getaffinity(0))
        share = len(cores) // world
        if share >= 4:  # a rank keeps four threads busy (its main thread and the planner's three)
            os.sched_setaffinity(0, cores[local * share:(local + 1) * share])
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    per_rank = {}

    def max_over_ranks(x: float, name: str) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        every = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        per_rank[name] = [round(float(v.item()) / args.steps * 1e3, 3) for v in every]
        return max(float(v.item()) for v in every)

    pk = peaks()
    coords_h, feats_h, sizes = make_batch(rank)
    cmax = coords_h[:, 1:].max(0).tolist()
    coords_pin = torch.from_numpy(coords_h).pin_memory()
    feats_pin = feats_h.pin_memory()
    coords_d = coords_pin.to(dev)
    feats_d = feats_pin.to(dev)
    torch.manual_seed(WEIGHT_SEED)
    model = pce.MinkUNet(IN_CHANNELS, NUM_CLASSES)
    pce.randomize_batchnorm(model, WEIGHT_SEED)
    model = model.half().eval().to(dev)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    logits_pin = torch.empty((len(coords_h), NUM_CLASSES), dtype=torch.float16).pin_memory()

    def tensor(c, f, ready=None):
        x = pce.spTensor(f, c, None, [0, 0, 0], cmax, batchsize=SCANS_PER_GPU, init_tag=pce.MinkUNet.tags())
        x.coords_ready = ready  # lets the map planner start as soon as the coordinates exist
        return x

    def step(c, f, ready=None):
        with torch.no_grad():
            return model(tensor(c, f, ready)).feats

    def steps_planned_one_ahead(n: int):
        """n forward passes, each preceded by the start of the NEXT pass's map construction
        (model.plan): every step holds one map construction and one forward pass, and the maps of a
        batch are being built while the batch before it computes.  The pass planned last is dropped."""
        nxt = tensor(coords_d, feats_d, resident)
        model.plan(nxt)
        for _ in range(n):
            flush.zero_()
            cur, nxt = nxt, tensor(coords_d, feats_d, resident)
            model.plan(nxt)
            with torch.no_grad():
                model(cur)

    resident = torch.cuda.Event()  # the device-resident inputs exist from here on
    resident.record()

    for _ in range(2):  # set-up, not warm-up: packs the weights, lets the planner create its storage
        step(coords_d, feats_d, resident)
        torch.cuda.synchronize()
    steps_planned_one_ahead(max(args.warmup, 3))
    # ---- device-resident timing ------------------------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.lib.pce_kernel_launches()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps_planned_one_ahead(args.steps)
    e1.record()
    barrier()
    dt = max_over_ranks(e0.elapsed_time(e1) * 1e-3, "ms_per_step")
    launches = int(_lib.lib.pce_kernel_launches() - launches0)
    # ---- the same K steps again with a CUDA-event pair around every convolution launch ------
    # (kept out of the loop above: ~80 extra event records per step perturb the headline time)
    PF.PROFILE = []
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    steps_planned_one_ahead(args.steps)
    p1.record()
    barrier()
    dt_prof = p0.elapsed_time(p1) * 1e-3
    prof, PF.PROFILE = PF.PROFILE, None
    # ---- end to end: pinned host -> device, forward, logits -> pinned host -----------------
    # A serving loop with two batches in flight: batch i's inputs are copied on an input stream (the
    # map planner starts on their arrival), its logits leave on an output stream, and the host waits
    # for batch i-1's logits once batch i is queued.  Every step moves its own inputs and its own
    # result; input and result buffers are double.
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    c_buf = [torch.empty_like(coords_d) for _ in range(2)]
    f_buf = [torch.empty_like(feats_d) for _ in range(2)]
    l_pin = [logits_pin, torch.empty_like(logits_pin).pin_memory()]
    ev_in = [torch.cuda.Event() for _ in range(2)]     # inputs of the batch are on the device
    ev_done = [torch.cuda.Event() for _ in range(2)]   # the batch is computed (its input buffers are free)
    ev_out = [torch.cuda.Event() for _ in range(2)]    # its logits are on the host
    outs = [None, None]                                # device logits, alive until their copy was waited for
    def upload(i: int):
        """Batch i's inputs leave for the device and its map construction is started."""
        b = i & 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_done[b])
            c_buf[b].copy_(coords_pin, non_blocking=True)
            f_buf[b].copy_(feats_pin, non_blocking=True)
            ev_in[b].record(s_in)
        x = tensor(c_buf[b], f_buf[b], ev_in[b])
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
            flush.zero_()
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

    serve(max(args.warmup, 3))  # warm-up of this loop's own streams and allocation pattern
    barrier()
    t0 = time.perf_counter()
    serve(args.steps)
    dt_e2e = max_over_ranks(time.perf_counter() - t0, "e2e_ms_per_step")
    clocks = sampler.stop() if rank == 0 else None
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
    t_min = t_min_convs / max(args.steps, 1)
    x_last = pce.spTensor(feats_d, coords_d, None, [0, 0, 0], cmax, batchsize=SCANS_PER_GPU, init_tag=pce.MinkUNet.tags())
    with torch.no_grad():
        maps = model(x_last).kmaps
    for km in maps.values():
        lookups = km.n_out * (km.kv - (1 if km.subm else 0))
        map_bytes = 28 * km.n_in + 12 * lookups + 4 * km.n_out * km.kv + (0 if km.subm else 16 * km.n_out)
        t_min += map_bytes / (pk["hbm_gbs"] * 1e9)
    del maps, x_last
    roof = None
    if by_kernel:
        name, k = max(by_kernel.items(), key=lambda kv: kv[1]["t"])
        ach = k["bytes"] / k["t"] / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                "traffic": None, "kernel": name, "launches_timed": k["n"], "avg_launch_us": k["t"] / k["n"] * 1e6,
                "share_of_step": k["t"] / (dt_prof if dt_prof > 0 else 1.0),
                "tensor_tflops": k["flops"] / k["t"] / 1e12, "tensor_frac": k["flops"] / k["t"] / 1e12 / pk["tflops"],
                "peak_source": pk["source"], "note": "sum of algorithmic bytes of every launch of this kernel in the "
                "K steps run right after the timed ones / sum of their CUDA-event durations",
                # DRAM bytes per launch of two of the step's launch shapes, from the ncu captures summarised under
                # profiles/ (the aggregate over a step's 43 launch shapes has no single capture, hence traffic = null)
                "traffic_captures": [
                    {"layer": "subm 3x3x3 96->96, 486551 rows", "algorithmic_bytes": 194.0e6, "dram_bytes": 211.0e6,
                     "profile": "profiles/conv_umma_subm3_96x96_lidar8.md"},
                    {"layer": "subm 3x3x3 256->256, 486551 rows", "algorithmic_bytes": 508.4e6, "dram_bytes": 756.4e6,
                     "profile": "profiles/conv_umma_other_shapes_lidar8.md"}]}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    layers, cpu = None, None
    if not args.lean:
        layers, _ = layer_table(dev, pk)
        cpu_v, cpu_dt, cores, sample = oracle_scans_per_s(0, 1, 1)
        cpu = {"value": cpu_v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    total_scans = SCANS_PER_GPU * world * args.steps
    line = {
        "metric": METRIC, "value": total_scans / dt, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "minkunet_lidar_batch8", "scans_per_gpu": SCANS_PER_GPU, "voxels_per_gpu": int(len(coords_h)),
                   "voxels_per_scan": sizes, "in_channels": IN_CHANNELS, "classes": NUM_CLASSES,
                   "widths": "32-32-64-128-256-256-128-96-96", "map_build": "inside the timed step (planner threads, own streams), started one batch ahead (model.plan)",
                   "e2e_loop": "two batches in flight: H2D on an input stream and the batch's map construction start while the batch before it computes, D2H on an output stream, host waits for the previous batch's logits",
                   "l2": "192 MiB memset between steps, inside the timed region", "accumulate": "fp32"},
        "e2e": {"value": total_scans / dt_e2e, "unit": UNIT,
                "h2d_bytes_per_step": int(coords_pin.numel() * 4 + feats_pin.numel() * 2),
                "d2h_bytes_per_step": int(logits_pin.numel() * 2), "ms_per_step": dt_e2e / args.steps * 1e3},
        "gpu_launches": launches,
        "roofline": roof,
        "network_roofline": {"t_min_ms": t_min * 1e3, "t_measured_ms": dt / args.steps * 1e3,
                             "frac": t_min / (dt / args.steps),
                             "note": "sum over the step's convolutions of max(bytes/copy bandwidth, flops/GEMM peak) "
                                     "plus its kernel maps' algorithmic bytes / copy bandwidth, over the measured step"},
        "kernels": {k: {"launches": v["n"], "ms": v["t"] * 1e3} for k, v in by_kernel.items()},
        "conv_shapes": [{"kernel": k[0], "n_out": k[1], "kv": k[2], "cin": k[3], "cout": k[4], "launches": v[0],
                         "us_per_launch": v[1] / v[0] * 1e6, "GB/s": v[2] / v[1] / 1e9, "TFLOP/s": v[3] / v[1] / 1e12}
                        for k, v in sorted(by_shape.items(), key=lambda kv: -kv[1][1])][:16],
        "layers": layers,
        "cpu_baseline": cpu,
        "clocks": clocks,
    }
    if world > 1:
        line["per_rank"] = {**per_rank, "host_cores": host_cores, "cores_per_rank": len(os.sched_getaffinity(0)),
                            "pinned": bool(args.pin)}
    print(json.dumps(line))
    if world > 1:
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
    ap.add_argument("--workload", type=str, default="minkunet", choices=["minkunet", "scene", "indoor"],
                    help="minkunet: batch of 8 LiDAR scans per GPU (default); scene: one 1.5 M-voxel scene in x-slabs")
    ap.add_argument("--no-pin", dest="pin", action="store_false",
                    help="multi-rank runs: do not give each rank its own share of the host cores "
                         "(8 ranks on 32 cores measured 14,477 scans/s with the shares, 13,863 without)")
    ap.add_argument("--lean", action="store_true",
                    help="skip the per-layer table and the CPU baseline (short runs under a profiler)")
    args = ap.parse_args()
    if args.workload == "scene":
        run_scene(args)
    elif args.workload == "indoor":
        run_indoor(args)
    elif args.layer is not None:
        run_layer(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
