#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path on B200.

A step is one full frame of the SCN UNet of the reference's model.py (InputLayer mode 4, SSC 3->32,
UNet planes [32..224] x reps 2 residual, BN+ReLU, OutputLayer, Linear 32->20) over one seeded
synthetic room of ~250k voxels: voxel hashing, all rulebooks, 53 submanifold convolutions, 6+6 strided
(de)convolutions, 65 BatchNorm+ReLU, 6 1x1 convolutions.  The metric is "active voxels/s
per SSC layer": the active sites summed over the 53 submanifold-convolution layers of the frame, divided
by the time of the whole frame (everything else is charged to it).  The incremental frame (5 % of the
voxels changed, reference semantics) is timed beside it and reported as ms/frame.

  value      inputs resident in HBM when the timed region starts
  e2e        the same through the public module API with pinned HOST inputs and a host read of the result
  roofline   the dominant kernel (the gather-GEMM of the level-0 32->32 submanifold convolution: the warp-level
             tf32 kernel), timed alone with CUDA events on the launching stream, L2 flushed between launches
  tcgen05    the same measurement for the tcgen05 kernel on a wide layer (128->128 on the room's sites),
             reported against the tensor roofline
  hash_build the grid build (voxel hash + site ranking + input rules) at 36k, 255k and 4M points
  cpu_baseline  the CPU restatement of the reference (oracle/) on this box's host cores, rank 0, N=1 only

N > 1 (torchrun, one rank per GPU): every rank runs its own seeded room, no data-path collective; the
step time is the max over ranks (weak scaling).

`--impl reference` times the CPU restatement of the reference on the same workload instead.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "ins-conv_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

METRIC = "active voxels/s per SSC layer (UNet frame); incremental ms/frame beside it"
UNIT = "voxel-layers/s"
PLANES = [32, 64, 96, 128, 160, 192, 224]
L2_NOTE = "no flush: one frame streams ~1.5 GB of activations and maps, far above the 126 MB L2"
WORKLOAD = "configs[2]: model.py SCN UNet, one synthetic room (~250k voxels, 2 cm, 8x8x3 m), full frame"


def build_model(scn, torch):
    class NaiveUNet(torch.nn.Module):  # same topology as the reference's model.py:9-26
        def __init__(self):
            torch.nn.Module.__init__(self)
            m = PLANES[0]
            self.sparseModel = scn.Sequential().add(
                scn.InputLayer(3, 4096, mode=4)).add(
                scn.SubmanifoldConvolution(3, 3, m, 3, False)).add(
                scn.UNet(3, 2, PLANES, True)).add(
                scn.BatchNormReLU(m)).add(
                scn.OutputLayer(3))
            self.linear = torch.nn.Linear(m, 20)

        def forward(self, x, increment=False):
            return self.linear(self.sparseModel(x, increment))
    torch.manual_seed(0)
    return NaiveUNet().eval()


def make_scene(seed, voxels):
    import numpy as np
    from insconv import synth
    coords = synth.room(seed, target=voxels)
    feats = synth.rgb(seed, coords.shape[0])
    new_c, pert = synth.sweep_frame(coords, frame=50, seed=seed)
    # 5 % of the sites change: new surface voxels plus 1 % perturbed colours
    want = int(0.05 * coords.shape[0])
    new_c = new_c[:max(want - pert.shape[0], 1)]
    rng = np.random.RandomState(seed + 99)
    inc_coords = np.concatenate([new_c, coords[pert]], 0)
    inc_feats = np.concatenate([synth.rgb(seed + 1, new_c.shape[0]),
                                feats[pert] + rng.normal(0, 0.05, (pert.shape[0], 3)).astype(np.float32)], 0)
    return coords, feats, inc_coords, inc_feats.astype(np.float32)


class ClockSampler(object):
    """SM clock and throttle reasons of one GPU, sampled while the timed legs run.  In-process NVML queries from a
    thread (a few tens of microseconds each, every 100 ms); `nvidia-smi -lms` as a subprocess is the fallback.  (The
    subprocess form perturbs what it watches: one of its queries landing in a 35 ms timed region doubled the region.)"""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index, mode="nvml"):
        self.index = index
        self.proc = None
        self.lines = []
        self.nvml = None
        self.samples = []  # (sm_mhz, max_mhz, reasons bitmask)
        self.query_ms = []  # host time of each sample taken by the thread
        self.running = False
        self.mode = mode  # nvml | smi | off

    def start(self):
        if self.mode == "off":
            return
        if self.mode == "nvml":
            try:
                import pynvml
                pynvml.nvmlInit()
                visible = os.environ.get("CUDA_VISIBLE_DEVICES")
                phys = self.index
                if visible:
                    ids = [v.strip() for v in visible.split(",") if v.strip()]
                    if self.index < len(ids) and ids[self.index].isdigit():
                        phys = int(ids[self.index])
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
                self.nvml = pynvml
                self._sample_nvml()  # the first query initialises the library's state for the device
                self.running = True
                self.thread = threading.Thread(target=self._loop_nvml, daemon=True)
                self.thread.start()
                # the sampling thread's own first queries (per-thread library state) must be over before anything
                # is timed: a slow first query holds a driver lock that kernel launches wait for
                t0 = time.time()
                while len(self.samples) < 3 and time.time() - t0 < 2.0:
                    time.sleep(0.02)
                return
            except Exception:
                self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # the tool's start-up (driver library initialisation, first query) must be over before anything is timed
            t0 = time.time()
            while not self.lines and time.time() - t0 < 5.0:
                time.sleep(0.05)
        except Exception:
            self.proc = None

    def _sample_nvml(self):
        n = self.nvml
        sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        reasons = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        self.samples.append((float(sm), float(mx), int(reasons)))

    def _timed_sample(self):
        t0 = time.perf_counter()
        self._sample_nvml()
        self.query_ms.append((time.perf_counter() - t0) * 1e3)

    def _loop_nvml(self):
        while self.running:
            try:
                self._timed_sample()
            except Exception:
                pass
            time.sleep(0.1)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.running = False
            self.thread.join(timeout=2)
            n = self.nvml
            names = {"hw_slowdown": n.nvmlClocksThrottleReasonHwSlowdown,
                     "hw_thermal_slowdown": n.nvmlClocksThrottleReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": n.nvmlClocksThrottleReasonSwThermalSlowdown,
                     "sw_power_cap": n.nvmlClocksThrottleReasonSwPowerCap}
            reasons = sorted(k for k, bit in names.items() if any(s[2] & bit for s in self.samples))
            sm = [s[0] for s in self.samples]
            mx = [s[1] for s in self.samples]
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                    "samples": len(sm), "reasons": reasons, "source": "nvml",
                    "slowest_query_ms": round(max(self.query_ms), 3) if self.query_ms else None}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock sampler available"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


def layer_bench(args, dev, hbm_peak, bf16_peak, peak_kind):
    """One submanifold convolution on the room, rulebook cached, through the C ABI: the 'active voxels/s per
    SSC layer' figure in isolation.  L2 is flushed between launches; each launch is timed with CUDA events."""
    import torch
    from insconv import cabi
    half = args.precision == "fp16" and cabi.lib().scn_weights_packable_f16(27, args.n_in, args.n_out) == 1
    prec = cabi.PREC_FP32 if args.precision == "fp32" else cabi.PREC_TF32
    coords, _, _, _ = make_scene(0, args.voxels)
    m = cabi.Metadata()
    n = m.input_layer_build(4096, torch.from_numpy(coords).to(dev), mode=4)
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(n, args.n_in, generator=g).to(dev)
    w = (torch.randn(27, args.n_in, args.n_out, generator=g) * (2.0 / (27 * args.n_in)) ** 0.5).to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if half:  # fp16 rows (as a BatchNorm in front of the layer writes them) and the fp16 weight pack
        import ctypes
        x = x.half()
        wp = torch.empty(cabi.lib().scn_packed_size_f16(27, args.n_in, args.n_out), dtype=torch.float16, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        cabi.call("scn_pack_weights_f16", cabi.ptr(w), 27, args.n_in, args.n_out, cabi.ptr(wp), stream)
        out = torch.empty(n, args.n_out, dtype=torch.float32, device=dev)
        fl = ctypes.c_double(0)

        def run():
            cabi.call("scn_ssc_forward", m.h, cabi.size3(4096), cabi.ptr(x), args.n_in, cabi.ptr(out), args.n_out, cabi.ptr(wp),
                      None, args.n_in, args.n_out, cabi.PREC_F16, stream, ctypes.byref(fl))
            return out, fl.value
    else:
        def run():
            return m.ssc_forward(4096, x, w, None, prec)
    out, madds = run()
    times = []
    for i in range(args.warmup + args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out, madds = run()
        e1.record()
        torch.cuda.synchronize()
        if i >= args.warmup:
            times.append(e0.elapsed_time(e1) * 1e-3)
    cabi.check_errors()
    t = sum(times) / len(times)
    pairs = madds / (args.n_in * args.n_out)
    s_in = 2.0 if half else 4.0  # bytes per input feature and per weight
    byts = s_in * n * args.n_in + 4.0 * n * args.n_out + 8.0 * pairs + s_in * 27 * args.n_in * args.n_out
    flops = 2.0 * madds
    hbm_bound = args.n_in <= 64
    tensor_peak = bf16_peak if half else bf16_peak / 2  # 16-bit operands: the measured dense bf16 peak; tf32: half of it
    return {"sites": int(n), "n_in": args.n_in, "n_out": args.n_out, "pairs": int(pairs), "us_per_launch": t * 1e6,
            "voxels_per_s": n / t, "GBps": byts / t / 1e9, "TFLOPs": flops / t / 1e12,
            "roofline": {"bound": "hbm" if hbm_bound else "tensor", "achieved": byts / t / 1e9 if hbm_bound else flops / t / 1e12,
                         "peak": hbm_peak if hbm_bound else tensor_peak, "unit": "GB/s" if hbm_bound else "TFLOP/s",
                         "frac": (byts / t / 1e9 / hbm_peak) if hbm_bound else (flops / t / 1e12 / tensor_peak),
                         "peak_kind": peak_kind, "algorithmic_bytes": byts, "algorithmic_flops": flops}}


def labels_bench(dev, coords, steps, warmup):
    """Label fusion behind the network (row f2 of the scope table): one frame's scores for every voxel of the room
    merged into the device-resident vote table (SCN.Result_3.update), scores and coordinates already on the GPU; beside
    it the CPU restatement of the reference's Result<3> on a 20,000-point sample (the reference's own comment puts its
    host loop at about 30 ms for 20,000 points, Metadata/resultHash.h:53-54)."""
    import numpy as np
    import torch
    import sparseconvnet as scn
    from oracle import scn_labels
    rng = np.random.RandomState(5)
    n = coords.shape[0]
    scores = torch.softmax(torch.from_numpy(rng.randn(n, 20).astype(np.float32)), 1).to(dev)
    pts = torch.from_numpy(np.ascontiguousarray(coords[:, :3])).to(dev)
    table = scn.SCN.Result_3(3.0)
    for _ in range(warmup):
        table.update(pts, scores)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = scn.SCN.launch_count()
    e0.record()
    for _ in range(steps):
        table.update(pts, scores)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / steps
    launches = (scn.SCN.launch_count() - l0) // steps
    q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    q0.record()
    labels = table.multiQuery(pts)
    q1.record()
    torch.cuda.synchronize()
    sample = 20000
    cpu = scn_labels.Result(3.0)
    c_np, s_np = coords[:sample, :3], scores[:sample].cpu().numpy()
    cpu.update(c_np, s_np)
    t0 = time.perf_counter()
    cpu.update(c_np, s_np)
    cpu_ms = (time.perf_counter() - t0) * 1e3
    assert np.array_equal(labels[:sample].numpy(), cpu.multiQuery(c_np)), "the GPU table and the CPU restatement disagree"
    # bytes that have to move: coordinates and scores in, (key, label, confidence) read and written once
    alg = n * (24 + 80 + 2 * 16)
    return {"voxels": int(n), "classes": 20, "update_us": us, "voxels_per_s": n / (us * 1e-6), "launches": int(launches),
            "GBps": alg / (us * 1e-6) / 1e9, "entries": int(table.size()),
            "multi_query_with_host_copy_us": q0.elapsed_time(q1) * 1e3,
            "cpu_port": {"points": sample, "ms": cpu_ms, "kind": "port (Python dictionary restatement of the reference's host loop)"}}


def configs01_bench(dev, steps, warmup):
    """BASELINE configs[0] and configs[1] as single-layer figures through the C ABI: one SubmanifoldConvolution 16->16,
    fp32, no bias, on the seeded boxes-and-spheres scene (seed 3: 50,208 voxels in 128^3), rulebook cached; then the same
    layer over frame t+1's changed sites (insert + re-draw) as the incremental operator, beside the full recompute of
    frame t+1.  L2 flushed between launches, CUDA events on the launching stream."""
    import numpy as np
    import torch
    from insconv import cabi, synth
    coords = synth.boxes_and_spheres(3)
    rng = np.random.RandomState(3)
    feats = rng.randn(coords.shape[0], 16).astype(np.float32)
    w = torch.from_numpy(synth.kaiming_uniform(rng, 27, 16, 16)).to(dev)
    nf = synth.next_frame(coords, feats, 3)
    t = lambda a: torch.from_numpy(a).to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed_us(fn):
        ts = []
        for i in range(warmup + steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= warmup:
                ts.append(e0.elapsed_time(e1) * 1e3)
        return sum(ts) / len(ts)

    m0 = cabi.Metadata()
    n0 = m0.input_layer_build(128, t(coords), mode=4)
    v0 = m0.input_forward(t(feats))
    out = {}
    for name, prec in (("fp32", cabi.PREC_FP32), ("tf32", cabi.PREC_TF32)):
        _, madds = m0.ssc_forward(128, v0, w, None, prec)
        us = timed_us(lambda: m0.ssc_forward(128, v0, w, None, prec))
        pairs = madds / 256.0
        byts = 4.0 * n0 * 16 * 2 + 8.0 * pairs + 4.0 * 27 * 256
        out["configs0_" + name] = {"sites": int(n0), "pairs": int(pairs), "us_per_launch": us, "voxels_per_s": n0 / (us * 1e-6),
                                   "GBps_algorithmic": byts / (us * 1e-6) / 1e9}
    m1, mf = cabi.Metadata(), cabi.Metadata()
    n1 = m1.input_layer_build(128, t(nf["new_coords"]), mode=4)
    nfull = mf.input_layer_build(128, t(nf["coords"]), mode=4)
    res = m1.incre_input_forward(m0, t(nf["new_feats"]), v0)
    vf = mf.input_forward(t(nf["feats"]))
    m1.incre_ssc_forward(m0, 128, res, w, v0)
    mf.ssc_forward(128, vf, w)
    us_inc = timed_us(lambda: m1.incre_ssc_forward(m0, 128, res, w, v0))
    us_full = timed_us(lambda: mf.ssc_forward(128, vf, w))
    out["configs1_fp32"] = {"changed_sites": int(n1), "changed_frac": n1 / float(n0), "incremental_us": us_inc,
                            "full_recompute_us": us_full, "sites_next_frame": int(nfull),
                            "semantics": "reference (insert + re-draw, residual on the changed sites)"}
    return out


def dram_traffic(kernel, workload, precision):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch from the ncu capture recorded in
    profiles/dram_traffic.txt (columns: kernel workload precision bytes commit source), or None when no capture of that
    kernel and workload is on record."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        for ln in f:
            f_ = ln.split()
            if len(f_) >= 4 and not ln.startswith("#") and f_[0] == kernel and f_[1] == workload and f_[2] == precision:
                return {"bytes": float(f_[3]), "commit": f_[4] if len(f_) > 4 else None, "source": f_[5] if len(f_) > 5 else None}
    return None


def hash_bench(dev, steps, warmup, sizes=("c1", "room", "building")):
    """Grid build (points -> ranked sites + input rules) through the C ABI, coordinates resident on the device.
    Algorithmic bytes: 32 per point in (int64 x,y,z,batch), 12 per site (coordinates out), 4 per point (point ->
    site); with the open-addressing table (filled on the first coordinate query, timed as build + one query of one
    coordinate) 8 per table slot more."""
    import torch
    from insconv import cabi, synth
    out = []
    for name in sizes:
        if name == "c1":
            c = synth.boxes_and_spheres(0)
            size = 128
        elif name == "room":
            c = synth.room(0)
            size = 4096
        else:
            c = synth.building(0, target=4000000)
            size = 4096
        import numpy as np
        c4 = np.concatenate([c, np.zeros((c.shape[0], 1), np.int64)], 1)
        d = torch.from_numpy(c4).to(dev)
        m = cabi.Metadata()

        probe = torch.zeros(4, 1, dtype=torch.int32, device=dev)

        def median_build(with_table=False):
            ts = []
            for i in range(warmup + steps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                n = m.input_layer_build(size, d, mode=4)
                if with_table:
                    m.query(size, probe)
                e1.record()
                torch.cuda.synchronize()
                if i >= warmup:
                    ts.append(e0.elapsed_time(e1) * 1e-3)
            return sorted(ts)[len(ts) // 2], n

        cabi.call("scn_set_build_ahead", 0, 0)  # the hash build alone: input scale, no neighbour map
        t, n = median_build()
        t_table, _ = median_build(True)
        # coordinate queries through the open-addressing table (teams of four lanes per probe sequence): every site's own
        # coordinates plus as many shifted by one voxel (about half of which miss)
        soa = torch.from_numpy(np.ascontiguousarray(np.concatenate([c4, c4 + np.array([1, 0, 0, 0])], 0).T.astype(np.int32))).to(dev)
        qts = []
        for i in range(warmup + steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            m.query(size, soa)
            e1.record()
            torch.cuda.synchronize()
            if i >= warmup:
                qts.append(e0.elapsed_time(e1) * 1e-3)
        t_query = sorted(qts)[len(qts) // 2]
        # the 3x3x3 rulebook (27 lookups per site in the ranking structure) of that grid, built on first request
        counts = np.zeros(27, dtype=np.int64)
        rts = []
        for i in range(warmup + steps):
            m.input_layer_build(size, d, mode=4)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            cabi.call("scn_ssc_rulebook", m.h, cabi.size3(size), counts.ctypes.data, None,
                      torch.cuda.current_stream().cuda_stream)
            e1.record()
            torch.cuda.synchronize()
            if i >= warmup:
                rts.append(e0.elapsed_time(e1) * 1e-3)
        t_rules, pairs = sorted(rts)[len(rts) // 2], int(counts.sum())
        cabi.call("scn_set_build_ahead", 1, 6)  # what a UNet frame pays: 7 scales with their rulebook maps
        t_all, _ = median_build()
        cabi.call("scn_set_build_ahead", -1, -1)
        cap = 16
        while cap < 2 * n:
            cap *= 2
        byts = 32.0 * c4.shape[0] + 12.0 * n + 4.0 * c4.shape[0]
        out.append({"scene": name, "points": int(c4.shape[0]), "sites": int(n), "us": t * 1e6,
                    "points_per_s": c4.shape[0] / t, "GBps": byts / t / 1e9,
                    "with_open_addressing_table": {"us": t_table * 1e6, "GBps": (byts + 8.0 * cap) / t_table / 1e9},
                    "table_query": {"queries": int(soa.shape[1]), "us": t_query * 1e6, "queries_per_s": soa.shape[1] / t_query},
                    "us_with_6_coarse_scales_and_all_maps": t_all * 1e6,
                    # algorithmic bytes of the rulebook build: coordinates in, occupied bitmap words and their
                    # prefixes read once (12 bytes per site at most), pairs out
                    "ssc_rulebook": {"pairs": pairs, "us": t_rules * 1e6,
                                     "GBps": (12.0 * n + 12.0 * n + 8.0 * pairs) / t_rules / 1e9}})
    return out


def slab_bench(args, rank, world, local, dist):
    """configs[4], second part: one 4M-voxel building split into x-slabs (one per GPU) with halo rows exchanged by
    grouped NCCL send/recv after every submanifold and strided convolution.  Strong scaling: the scene is fixed."""
    import numpy as np
    import torch
    import sparseconvnet as scn
    from insconv import slab, synth
    dev = torch.device("cuda", local)
    scn.set_precision(args.precision)
    model = build_model(scn, torch).to(dev)
    coords = synth.building(0, target=args.voxels if args.voxels > 1000000 else 4000000)
    feats = synth.rgb(0, coords.shape[0])
    align = 2 ** (len(PLANES) - 1)
    cuts = slab.cuts_balanced(coords[:, 0], world, align)
    ext = slab.load_mask(coords, cuts, rank, len(PLANES))
    n_own = int(slab.owned_mask(coords[:, 0], cuts, rank).sum())
    peer = world > 1 and args.halo == "peer"
    ex = slab.PeerSlabExchange(dist, rank, world, cuts, 4096, dev) if peer else slab.SlabExchange(dist, rank, world, cuts, 4096)
    if world > 1:
        slab.install(model, ex)
    dc, df = torch.from_numpy(coords[ext]).to(dev), torch.from_numpy(feats[ext]).to(dev)

    def frame():
        return model([dc, df])

    if peer:  # one untimed frame with the pushed bytes summed on the device
        ex.track_bytes = True
        frame()
        ex.track_bytes = False
        sent_one_frame, ex_one_frame = ex.bytes_sent, ex.exchanges
    for _ in range(args.warmup):
        frame()
    if peer:
        ex.check()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = scn.SCN.launch_count()
    e0.record()
    for _ in range(args.steps):
        frame()
    e1.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    launches = scn.SCN.launch_count() - l0
    if peer:
        ex.check()  # raises if a neighbour did not answer or a plane did not fit its slot
        frames = 1
        sent_total, n_ex = sent_one_frame, ex_one_frame
    else:
        frames = max(args.steps + args.warmup, 1)
        sent_total, n_ex = ex.bytes_sent, ex.exchanges
    ssc_mods = [m for m in model.modules() if isinstance(m, scn.SubmanifoldConvolution)]
    layers_local = sum(int(m.save_input_feats.shape[0]) for m in ssc_mods)
    if dist is not None:
        t = torch.tensor([ms, float(layers_local), float(sent_total)], device=dev, dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, layers_all, sent = float(tmax[0]), float(t[1]), float(t[2])
    else:
        layers_all, sent = float(layers_local), 0.0
    if rank == 0:
        # the unit counts rows entering the 53 submanifold convolutions of the UNDIVIDED scene: sites per level of the
        # whole building (built once here, outside the timed region) times the layers that run on each level
        from insconv import cabi

        def per_level(c):
            m = cabi.Metadata()
            counts, size = [int(m.input_layer_build(4096, c, mode=4))], 4096
            for _ in range(len(PLANES) - 1):
                n_out = ctypes.c_int64(0)
                cabi.call("scn_conv_prepare", m.h, cabi.size3(size), cabi.size3(size // 2), torch.cuda.current_stream().cuda_stream,
                          ctypes.byref(n_out))
                counts.append(int(n_out.value))
                size //= 2
            return counts
        local_counts, whole_counts = per_level(dc), per_level(torch.from_numpy(coords).to(dev))
        whole_layers = sum(whole_counts[local_counts.index(int(m.save_input_feats.shape[0]))] for m in ssc_mods)
        print(json.dumps({"metric": METRIC, "value": whole_layers / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None,
                          "dtype": {"fp32": "f32", "tf32": "tf32", "fp16": "f16"}[args.precision], "data": "synthetic",
                          "config": {"workload": "configs[4] part 2: one %d-voxel building (5 rooms x 4 floors) in %d x-slabs, "
                                                 "halo rows exchanged after every SSC / strided convolution"
                                                 % (coords.shape[0], world),
                                     "cuts": cuts, "ghost_zone": "per level, the plane next to each cut (coarse cells by one point each)",
                                     "voxel_layers_of_the_whole_scene": whole_layers,
                                     "voxel_layers_computed_incl_ghost": layers_all,
                                     "halo": "rows pushed into the neighbour's memory by the library's own kernels (CUDA IPC "
                                             "over NVLink), no NCCL call in the frame" if peer else "NCCL grouped send/recv",
                                     "halo_bytes_sent_per_frame": sent / frames,
                                     "exchanges_per_frame": n_ex // frames},
                          "gpu_launches": int(launches)}))


def rooms_bench(args, rank, world, local, dist):
    """configs[4], first part: 64 independent seeded rooms, scene i on rank i % world (insconv.shard), every rank with its
    own model copy and one Metadata per scene; no data-path collective.  A step runs every room once; strong scaling
    (the batch is fixed)."""
    import torch
    import sparseconvnet as scn
    from insconv import shard, synth
    dev = torch.device("cuda", local)
    scn.set_precision(args.precision)
    model = build_model(scn, torch).to(dev)
    n_scenes = 64
    mine = shard.scenes_for_rank(n_scenes, rank, world)
    scenes = []
    for i in mine:
        c = synth.room(i, target=args.voxels)
        scenes.append((torch.from_numpy(c).to(dev), torch.from_numpy(synth.rgb(i, c.shape[0])).to(dev)))
    voxels = sum(int(c.shape[0]) for c, _ in scenes)
    ssc_mods = [m for m in model.modules() if isinstance(m, scn.SubmanifoldConvolution)]
    layers = 0  # rows entering the 53 submanifold convolutions, summed over this rank's rooms (the bench's unit)
    for c, f in scenes:
        model([c, f])
        layers += sum(int(m.save_input_feats.shape[0]) for m in ssc_mods)

    def step():
        for c, f in scenes:
            model([c, f])

    for _ in range(args.warmup):
        step()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = scn.SCN.launch_count()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    launches = scn.SCN.launch_count() - l0
    total_voxels, _ = shard.aggregate(dist, dev, voxels, ms)
    total_layers, ms = shard.aggregate(dist, dev, layers, ms)
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": total_layers / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None,
                          "dtype": {"fp32": "f32", "tf32": "tf32", "fp16": "f16"}[args.precision], "data": "synthetic",
                          "config": {"workload": "configs[4] part 1: 64 seeded rooms (~%d voxels each), scene i on rank i %% %d, "
                                                 "one full UNet frame per room per step" % (args.voxels, world),
                                     "scenes": n_scenes, "voxels_total": int(total_voxels), "voxel_layers_total": int(total_layers),
                                     "ms_per_room": ms * world / n_scenes},
                          "gpu_launches": int(launches)}))


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def cpu_reference(voxels, steps, warmup, seed=0):
    """The CPU restatement of the reference (oracle/) on the host cores: full UNet frame on a room.  The module tree
    comes from the oracle's own topology builder, so this leg never loads the CUDA library."""
    import torch
    torch.set_num_threads(os.cpu_count())
    from oracle import scn_topology
    from oracle.scn_graph import GraphRunner
    torch.manual_seed(0)
    model = scn_topology.Naive_UNet().eval()
    coords, feats, _, _ = make_scene(seed, voxels)
    x = [torch.from_numpy(coords), torch.from_numpy(feats)]
    times, layers = [], 0
    for i in range(warmup + steps):
        runner = GraphRunner(model)
        t0 = time.perf_counter()
        runner._run(model.linear, runner._run(model.sparseModel, x, False), False)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        layers = voxel_layers_of(runner)
    t = sum(times) / len(times)
    return {"value": layers / t, "ms_per_step": t * 1e3, "voxels": int(coords.shape[0]), "voxel_layers": layers,
            "cores": os.cpu_count()}


def voxel_layers_of(runner):
    total = 0
    # the oracle runner keeps the input tensor of every SubmanifoldConvolution it evaluated
    for m in runner.root.modules():
        if type(m).__name__ == "SubmanifoldConvolution" and id(m) in runner.saved:
            total += int(runner.saved[id(m)].features.shape[0])
    return total


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--voxels", type=int, default=250000)
    ap.add_argument("--precision", default="fp16", choices=["fp32", "tf32", "fp16"])
    ap.add_argument("--quick", action="store_true", help="skip the 4M-point hash build (profiling aid)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--legs", default="full,incre,sweep,e2e,precisions,configs01,labels", help="which timed legs to run (profiling aid)")
    ap.add_argument("--sweep-frames", type=int, default=100)
    ap.add_argument("--no-build-overlap", action="store_true", help="value leg: grid builds on the frame's own stream")
    ap.add_argument("--layer", action="store_true", help="time one SSC layer alone (rulebook cached) and exit")
    ap.add_argument("--hash", action="store_true", help="time the grid build alone and exit")
    ap.add_argument("--workload", default="room", choices=["room", "building", "rooms64"],
                    help="room: one scene per GPU (default); building: one 4M-voxel scene split into x-slabs; "
                         "rooms64: 64 rooms shared out over the GPUs")
    ap.add_argument("--halo", default="peer", choices=["peer", "nccl"],
                    help="building workload: how halo rows travel (own kernels into peer memory, or NCCL send/recv)")
    ap.add_argument("--n-in", type=int, default=32)
    ap.add_argument("--n-out", type=int, default=32)
    ap.add_argument("--profile", action="store_true", help="allow fewer than 3 warm-up steps (numbers are not bench values)")
    ap.add_argument("--clock-sampler", default="nvml", choices=["nvml", "smi", "off"],
                    help="how SM clocks and throttle reasons are sampled during the timed legs: in-process NVML queries "
                         "(default), an nvidia-smi subprocess, or not at all")
    ap.add_argument("--no-gc-freeze", action="store_true",
                    help="leave Python's cyclic collector alone (by default the objects that exist after the first frame are "
                         "frozen out of it, as a long-running service does after start-up)")
    args = ap.parse_args()
    if args.impl == "b200" and not args.profile:
        args.warmup = max(args.warmup, 3)
    legs = set(args.legs.split(","))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return 0
        # the same room as the GPU arm, exactly K timed steps after W warm-up steps (a frame is about 1.5 s on 16 cores)
        r = cpu_reference(args.voxels, max(1, args.steps), max(0, args.warmup))
        line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": max(1, args.steps), "warmup": max(0, args.warmup), "ms_per_step": r["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": {"workload": WORKLOAD, "voxels_per_scene": r["voxels"], "scenes": 1,
                                                "voxel_layers_per_scene": r["voxel_layers"], "l2": L2_NOTE},
                "precision": {"name": "fp32", "note": "torch CPU fp32 (index_select -> mm -> index_add_ per offset)"},
                "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                                 "sample": "every step is one full UNet frame on the %d-voxel room of the GPU arm, torch CPU "
                                           "threads = cores" % r["voxels"]},
                "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    import numpy as np
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this library has no CPU fallback"}))
        return 1
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "rooms64":
        rooms_bench(args, rank, world, local, dist)
        if dist is not None:
            dist.destroy_process_group()
        return 0
    if args.workload == "building":
        slab_bench(args, rank, world, local, dist)
        if dist is not None:
            dist.destroy_process_group()
        return 0
    if args.hash:
        print(json.dumps({"hash_build": hash_bench(dev, args.steps, args.warmup, ("c1", "room") if args.quick else ("c1", "room", "building"))}))
        return 0
    if args.layer:
        hbm_peak, bf16_peak, peak_kind = load_peaks()
        print(json.dumps({"layer": layer_bench(args, dev, hbm_peak, bf16_peak, peak_kind), "precision": args.precision}))
        return 0
    import sparseconvnet as scn
    scn.set_precision(args.precision)
    model = build_model(scn, torch).to(dev)
    coords, feats, inc_c, inc_f = make_scene(rank, args.voxels)
    d_coords, d_feats = torch.from_numpy(coords).to(dev), torch.from_numpy(feats).to(dev)
    d_inc_c, d_inc_f = torch.from_numpy(inc_c).to(dev), torch.from_numpy(inc_f).to(dev)
    h_coords, h_feats = torch.from_numpy(coords).pin_memory(), torch.from_numpy(feats).pin_memory()
    hbm_peak, bf16_peak, peak_kind = load_peaks()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def per_rank(ms):
        if dist is None:
            return [round(ms, 4)]
        t = torch.zeros(world, device=dev, dtype=torch.float64)
        t[rank] = ms
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return [round(float(v), 4) for v in t.tolist()]

    def sum_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([float(v)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    REGIONS = 3

    def timed(fn, steps, warmup, before_region=None, end_of_region=None):
        """W warm-up steps, then REGIONS timed regions of exactly K steps each (barrier + device synchronisation on
        both sides, CUDA events, maximum over ranks).  The figure returned is the median region: single steps of
        10-100 ms that have nothing to do with the kernels (the whole virtual machine pauses; see step_host_ms) land
        in about one region out of three on this pool and would otherwise decide the result.  Every region's figure
        is kept in the JSON line (ms_per_step_of_each_region)."""
        for _ in range(warmup):
            fn()
        if end_of_region is not None:
            end_of_region()
        regions = []
        for _ in range(REGIONS):
            if before_region is not None:
                before_region()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = scn.SCN.launch_count()
            stamps = [time.perf_counter()]
            e0.record()
            for _ in range(steps):
                fn()
                stamps.append(time.perf_counter())  # host side only: when each step's launches had been queued
            if end_of_region is not None:
                end_of_region()  # work the steps left in flight (the e2e leg's last host read) belongs to the region
            e1.record()
            barrier()
            host_ms = [(b - a) * 1e3 for a, b in zip(stamps, stamps[1:])]
            mine = e0.elapsed_time(e1) / steps
            regions.append({"ms": max_over_ranks(mine), "by_rank": per_rank(mine),
                            "launches": (scn.SCN.launch_count() - l0) // steps,
                            "host": {"median": round(statistics.median(host_ms), 3), "max": round(max(host_ms), 3),
                                     "max_at_step": host_ms.index(max(host_ms))}})
        pick = sorted(regions, key=lambda r: r["ms"])[len(regions) // 2]
        step_host_ms.append(pick["host"])
        ms_by_rank.append(pick["by_rank"])
        region_ms.append([round(r["ms"], 4) for r in regions])
        return pick["ms"], pick["launches"]

    region_ms = []  # per timed leg: ms per step of each of its regions (the reported one is their median)
    ms_by_rank = []  # per timed leg: every rank's own ms per step (the reported figure is the maximum)
    step_host_ms = []  # one entry per timed leg, in the order full, incremental, exact, e2e

    # ---- value: full frame, inputs resident in HBM ------------------------------------------------
    out_holder = {}

    def full_frame():
        out_holder["y"] = model([d_coords, d_feats])

    full_frame()
    torch.cuda.synchronize()
    # Python's cyclic collector: a frame creates ~1000 container objects, so a full (oldest-generation) collection
    # comes round every ~100 frames and then walks every object torch and numpy have created since import, 30-80 ms
    # with the interpreter lock held.  Freezing what exists now keeps those walks short, as a long-running service
    # would do after start-up (--no-gc-freeze leaves the collector alone).
    if not args.no_gc_freeze:
        import gc
        gc.collect()
        gc.freeze()
    ssc_mods = [m for m in model.modules() if isinstance(m, scn.SubmanifoldConvolution)]
    voxel_layers = sum(int(m.save_input_feats.shape[0]) for m in ssc_mods)
    sampler = ClockSampler(local, args.clock_sampler)
    if rank == 0:
        sampler.start()
    # inputs are resident: the next frame's grid build may overlap this frame's last layers (a stream of its own)
    if not args.no_build_overlap:
        scn.overlap_grid_build(True)
    ms_full, launches = timed(full_frame, args.steps, args.warmup)
    scn.overlap_grid_build(False)
    total_layers = sum_over_ranks(voxel_layers)
    value = total_layers / (ms_full * 1e-3)

    # ---- incremental frame (reference semantics) against the saved full frame -----------------------
    def incre_frame():
        out_holder["y1"] = model([d_inc_c, d_inc_f], True)

    ms_incre, launches_incre = timed(incre_frame, args.steps, args.warmup) if "incre" in legs else (float("nan"), 0)

    def sites_per_level(c):
        from insconv import cabi
        m = cabi.Metadata()
        counts = [int(m.input_layer_build(4096, c, mode=4))]
        size = 4096
        for _ in range(len(PLANES) - 1):
            n_out = ctypes.c_int64(0)
            cabi.call("scn_conv_prepare", m.h, cabi.size3(size), cabi.size3(size // 2), torch.cuda.current_stream().cuda_stream,
                      ctypes.byref(n_out))
            counts.append(int(n_out.value))
            size //= 2
        return counts

    # fraction of the sites of each scale that the incremental frame computes on
    lv_full, lv_inc = sites_per_level(d_coords), sites_per_level(d_inc_c)
    recomputed = [round(a / max(b, 1), 4) for a, b in zip(lv_inc, lv_full)]

    # ---- exact incremental frame: the new points are merged into the kept scene and the merged scene is
    # recomputed (equals a full recompute; the kept scene advances each frame)
    def exact_frame():
        out_holder["y2"] = model([d_inc_c, d_inc_f], "exact")

    # every region starts from the base room again: the kept scene grows with each exact frame
    ms_exact, _ = timed(exact_frame, args.steps, args.warmup, before_region=full_frame) if "incre" in legs else (float("nan"), 0)

    # ---- online sequence (configs[3]): seeded camera sweep, one insertion of 2-8 % new surface voxels per frame.
    # Pass 1, reference semantics: every frame is a residual update against the last full frame; every 10th frame the
    # accumulated scene is recomputed in full (which renews the saved state).  Pass 2, exact mode: every frame merges
    # its points into the kept scene and recomputes it (the kept scene advances by itself).
    sweep = None
    if "sweep" in legs and world == 1:
        from insconv import synth
        import numpy as np
        n_frames = args.sweep_frames
        frames = []
        for fr in range(n_frames):
            nc, _ = synth.sweep_frame(coords, fr, n_frames=n_frames, seed=rank)
            frames.append((torch.from_numpy(nc).to(dev), torch.from_numpy(synth.rgb(1000 + fr, nc.shape[0])).to(dev)))

        def clocked(fn):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) * 1e3

        lat = {"reference": [], "full": [], "exact": []}
        model([d_coords, d_feats])  # the last full frame: the base room
        acc_c, acc_f = [d_coords], [d_feats]
        for fr, (dn, dfn) in enumerate(frames):
            lat["reference"].append(clocked(lambda: model([dn, dfn], True)))
            acc_c.append(dn)
            acc_f.append(dfn)
            if fr % 10 == 9:
                all_c, all_f = torch.cat(acc_c), torch.cat(acc_f)
                lat["full"].append(clocked(lambda: model([all_c, all_f])))
        scene_points_reference = int(sum(c.shape[0] for c in acc_c))
        model([d_coords, d_feats])
        model(list(frames[0]), "exact")  # untimed: first use of the exact mode (one-time set-up, as every timed leg warms up)
        model([d_coords, d_feats])  # reset the kept scene to the base room
        worst = (0.0, -1)
        for fr, (dn, dfn) in enumerate(frames):
            lat["exact"].append(clocked(lambda: model([dn, dfn], "exact")))
            if lat["exact"][-1] > worst[0]:
                worst = (lat["exact"][-1], fr)
        pct = lambda v, q: float(sorted(v)[min(len(v) - 1, int(q * len(v)))])
        stats = lambda v: {"mean": sum(v) / len(v), "p50": pct(v, 0.5), "p99": pct(v, 0.99)}
        sweep = {"frames": n_frames,
                 "scene_voxels_at_end": int(model.sparseModel[0].scene_coords.shape[0]),
                 "reference_ms": stats(lat["reference"]),
                 "full_recompute_every_10th_frame_ms": stats(lat["full"]),
                 "exact_ms": stats(lat["exact"]), "exact_slowest_frame": {"ms": worst[0], "frame": worst[1]},
                 "points_fed_in_reference_pass": scene_points_reference,
                 "timing": "host wall clock around each frame, device synchronised on both sides"}
        model([d_coords, d_feats])

    # ---- e2e: pinned host inputs, host read of the result -------------------------------------------
    # As a serving loop would run it: one frame in flight.  Step t queues its input copies and its frame, hands the
    # result to a copy stream (device -> pinned host, double-buffered) and only then waits for the result of step t-1
    # and reads it; every step's result reaches the host and is read, the last one inside the timed region (timed()
    # synchronises the device before it stops the clock and drain() reads what is left).
    h_outs = [torch.empty(coords.shape[0], 20, dtype=torch.float32).pin_memory() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    copied = [torch.cuda.Event(), torch.cuda.Event()]
    e2e_state = {"t": 0, "pending": None, "checksum": 0.0}

    def e2e_read(i):
        copied[i].synchronize()
        e2e_state["checksum"] += float(h_outs[i][0, 0]) + float(h_outs[i][-1, -1])  # the host touches the result

    def e2e_frame():
        i = e2e_state["t"] & 1
        y = model([h_coords, h_feats.to(dev, non_blocking=True)])
        done = torch.cuda.Event()
        done.record()
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(done)
            h_outs[i].copy_(y, non_blocking=True)
            copied[i].record()
        y.record_stream(copy_stream)
        if e2e_state["pending"] is not None:
            e2e_read(e2e_state["pending"])
        e2e_state["pending"] = i
        e2e_state["t"] += 1

    def e2e_drain():
        if e2e_state["pending"] is not None:
            e2e_read(e2e_state["pending"])
            e2e_state["pending"] = None

    ms_e2e, _ = timed(e2e_frame, args.steps, args.warmup, end_of_region=e2e_drain) if "e2e" in legs else (float("nan"), 0)
    # the same full frame in the other precisions (fewer steps: these are reported beside the headline, not as it)
    other = {}
    if "precisions" in legs:
        for prec in ("fp16", "tf32", "fp32"):
            if prec == args.precision:
                continue
            scn.set_precision(prec)
            ms_p, launches_p = timed(full_frame, min(args.steps, 20), 3)
            other[prec] = {"ms_per_step": ms_p, "value": total_layers / (ms_p * 1e-3), "launches": int(launches_p)}
        scn.set_precision(args.precision)
        full_frame()
    clocks = sampler.stop() if rank == 0 else None  # sampled across the timed legs
    e2e_value = total_layers / (ms_e2e * 1e-3)
    h2d = coords.nbytes + feats.nbytes
    d2h = int(out_holder["y"].numel()) * 4

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0

    # roofline of the dominant kernel: the level-0 submanifold convolution (32 -> 32 planes on every site of the
    # room), timed alone with CUDA events on its stream, L2 flushed between launches
    args.n_in, args.n_out = 32, 32
    lay = layer_bench(args, dev, hbm_peak, bf16_peak, peak_kind)
    roofline = dict(lay["roofline"])
    roofline.update({"kernel": "gather-GEMM %s (%s), SSC 32->32 on %d sites (level 0 of the UNet: 9 of the 53 SSC "
                               "layers, 78 %% of the frame's voxel-layers)"
                               % (args.precision, "FFMA kernel" if args.precision == "fp32" else "warp-level mma.sync kernel",
                                  lay["sites"]),
                     "us_per_launch": lay["us_per_launch"], "voxels_per_s": lay["voxels_per_s"],
                     "traffic": None,
                     "l2": "flushed between launches (256 MB write)"})
    tr = dram_traffic("gather_mma_warp", "ssc32_room_%d" % args.voxels, args.precision)
    if tr:
        roofline.update({"traffic": tr["bytes"], "traffic_from": tr})
    tcgen05 = None
    if args.precision != "fp32":  # the tcgen05 kernel on a wide layer, against the tensor roofline
        args.n_in, args.n_out = 128, 128
        wide = layer_bench(args, dev, hbm_peak, bf16_peak, peak_kind)
        tcgen05 = dict(wide["roofline"])
        tcgen05.update({"kernel": "gather-GEMM %s (tcgen05 persistent kernel), SSC 128->128 on %d sites"
                                  % ("fp16 rows, kind::f16" if args.precision == "fp16" else "tf32", wide["sites"]),
                        "us_per_launch": wide["us_per_launch"],
                        "peak_note": "fp16: the measured dense bf16 peak; tf32: half of it (tf32 is not in MEASURED_PEAKS.json)",
                        "traffic": None})
        tr = dram_traffic("gather_gemm_tc_persist", "ssc128_room_%d" % args.voxels, args.precision)
        if tr:
            tcgen05.update({"traffic": tr["bytes"], "traffic_from": tr})
    hashes = hash_bench(dev, 5, 2, ("c1", "room") if args.quick else ("c1", "room", "building"))
    for h in hashes:
        h["hbm_frac"] = h["GBps"] / hbm_peak
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_full, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"fp32": "f32", "tf32": "tf32", "fp16": "f16"}[args.precision], "data": "synthetic",
            "config": {"workload": WORKLOAD, "voxels_per_scene": int(coords.shape[0]), "scenes": world,
                       "voxel_layers_per_scene": voxel_layers, "l2": L2_NOTE,
                       "grid_build": ("on the frame's stream" if args.no_build_overlap else
                                      "value leg: on a second stream, overlapping the previous frame's last layers "
                                      "(inputs resident); every other leg on the frame's stream")},
            "precision": {"name": args.precision,
                          "note": {"fp32": "fp32 FFMA throughout",
                                   "tf32": "fp32 tensors, tensor cores read them as tf32, fp32 accumulation",
                                   "fp16": "BatchNorm hands fp16 rows to the convolution behind it (fp16 x fp16 products, "
                                           "fp32 accumulation and fp32 outputs); layers without a BatchNorm in front (first "
                                           "layer, 1x1 shortcuts) read fp32 as tf32"}[args.precision]},
            "incremental": {"ms_per_frame": ms_incre, "changed_points": int(inc_c.shape[0]),
                            "changed_frac": float(inc_c.shape[0]) / coords.shape[0],
                            "semantics": "reference (insert-only, no dilation)", "launches": int(launches_incre),
                            "sites_per_level": lv_inc, "fraction_of_full_frame_sites_per_level": recomputed},
            "incremental_exact": {"ms_per_frame": ms_exact,
                                  "semantics": "new points merged into the kept scene, merged scene recomputed: "
                                               "equal to a full recompute, kept scene advances"},
            "sweep": sweep,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h),
                    "pipelining": "one frame in flight: the host waits for and reads step t-1's result (pinned, copied on "
                                  "a second stream) after queueing step t; every step's result is read, the last inside "
                                  "the timed region"},
            "gpu_launches": int(launches) * args.steps,
            # host time between the ends of consecutive steps of each timed leg (full, incremental, exact, e2e as
            # run): a single step far above the median is a stall of the host or the driver, not of the kernels
            "step_host_ms": step_host_ms, "ms_per_step_by_rank": ms_by_rank,
            "timing": {"regions_per_leg": REGIONS, "steps_per_region": args.steps, "reported": "median region",
                       "ms_per_step_of_each_region": region_ms, "legs": "full, incremental, exact, e2e as run"},
            "clocks": clocks, "roofline": roofline, "tcgen05": tcgen05,
            "hash_build": hashes,
            # the same frame in the other precisions, value and ms per step (median of 3 regions of min(K, 20) steps)
            "other_precisions": other,
            "single_layer": configs01_bench(dev, 20, 3) if "configs01" in legs else None,
            "label_fusion": labels_bench(dev, coords, 20, 3) if "labels" in legs else None}
    if world == 1 and not args.no_cpu_baseline:
        r = cpu_reference(args.voxels, 3, 1)
        line["cpu_baseline"] = {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                                "ms_per_step": r["ms_per_step"],
                                "sample": "3 full UNet frames (after 1 warm-up frame) on the same %d-voxel room, "
                                          "torch CPU threads = cores" % r["voxels"]}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
