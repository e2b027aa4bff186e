"""Benchmark of the sparse-filter convolution path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload vgg19] [--batch 16]
    python bench.py --impl reference ...        # the reference's CPU path on the host cores

A step is one pass over one batch: every conv layer of the workload launched back to back, each
on its own synthetic input that already sits in HBM.  The metric is whole-job images/s (batch *
ranks / step time); ms_per_step is the per-model sum-of-layers sparse-conv latency the
reference reports (evalution/overall_speedup.py:159-165).  One JSON line goes to stdout.

Multi-GPU: one process per GPU (torchrun); each rank runs its own batch on its own device
(independent batch shards, no collective on the data path), the step time is the max over
ranks.  `value` is the weak-scaling figure (a fixed batch per GPU); the `strong` block of the
same line is one global batch cut into per-rank slices by the batch partitioner.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402


# DRAM traffic of a kernel, from one ncu capture each (dram__bytes_read.sum + dram__bytes_write.sum
# of a launch over the algorithmic bytes of the captured layer); the bench scales it to its own
# mean launch.  The captures are summarised under profiles/.
NCU_TRAFFIC = {
    "tensor16_3x3_s1": {"dram_over_algorithmic": 67.9 / 107.5,
                        "note": "captured on VGG-19 conv3_3 batch 16: 67.9 MB per launch against 107.5 MB "
                                "algorithmic (outputs still in L2 at kernel end); scaled by algorithmic bytes"},
    "tensor_3x3_s1": {"dram_over_algorithmic": 65.7 / 107.5,
                      "note": "captured on VGG-19 conv3_3 batch 16: 65.7 MB per launch against 107.5 MB "
                              "algorithmic (outputs still in L2 at kernel end); scaled by algorithmic bytes"},
    "tiled_3x3_s1": {"dram_over_algorithmic": 270.5 / 205.7,
                     "note": "captured on VGG-19 conv2_2 batch 16: 270.5 MB per launch against 205.7 MB "
                             "algorithmic; scaled by algorithmic bytes"},
}
VARIANT_NAMES = {0: "auto", 1: "generic", 2: "tiled", 4: "tensor", 5: "tensor16"}
ARITH = {"tensor16": "3xFP16 split on the tensor cores (x_hi*w_hi + x_lo*w_hi + x_hi*w_lo, 11-bit halves), FP32 "
                     "accumulate, partial sums added on the CUDA cores every 48 MMAs; out-of-range activations "
                     "recomputed in 3xTF32",
         "tensor": "3xTF32 split on the tensor cores (x_hi*w_hi + x_lo*w_hi + x_hi*w_lo), FP32 accumulate, "
                   "partial sums added on the CUDA cores every 48 MMAs",
         "tiled": "FP32 FMA on the CUDA cores, taps added in the reference's (ic, r, s) order",
         "generic": "FP32 FMA on the CUDA cores", "depthwise": "FP32 FMA on the CUDA cores"}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def oracle_module():
    """The CPU oracle: the checker of the timed outputs and the CPU baseline, never a compute path."""
    from oracle import oracle as orc
    return orc


class ClockSampler:
    """Samples nvidia-smi clocks, power and throttle reasons while a timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, pw, reasons = [], [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2])); pw.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "power_w_median": float(np.median(pw)) if pw else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm)}


class Model:
    """The conv layers of one workload on one GPU: compressed filters, NHWC inputs and outputs
    sized for `max_batch` (smaller batches use the leading images of the same buffers)."""

    def __init__(self, tb, wl, torch, workload, max_batch, device, oc_block=0, tile_ic=0, variant=0,
                 plan_cache=None):
        self.tb, self.wl, self.torch, self.name, self.max_batch = tb, wl, torch, workload, max_batch
        self.layers, self.tuned = [], set()
        for idx, L in enumerate(wl.WORKLOADS[workload]()):
            filt = wl.make_filter(workload, idx, L)
            path = os.path.join(plan_cache, "%s_%02d_%s.tetris" % (workload, idx, L.name)) if plan_cache else None
            loaded = bool(path and os.path.exists(path))
            if loaded:
                f = tb.SparseFilter.load(path, device=device)   # compressed forms + tuned tile plans
            else:
                f = tb.SparseFilter(filt, L.IC, L.OC, L.KS, TILE_IC=tile_ic, groups=L.groups, device=device,
                                    oc_block=oc_block)
            oh, ow = wl.out_extent(L.H, L.KS, L.stride, L.pad), wl.out_extent(L.W, L.KS, L.stride, L.pad)
            g = torch.Generator(device="cuda").manual_seed(1000 + idx)
            x = torch.rand(max_batch, L.H, L.W, L.IC, device="cuda", generator=g)
            x = x * (torch.rand(x.shape, device="cuda", generator=g) >= 0.5)
            y = torch.empty(max_batch, oh, ow, L.OC, device="cuda")
            self.layers.append(dict(L=L, f=f, x=x, y=y, oh=oh, ow=ow, nnz=int(f.nnz_), filt=filt,
                                    variant=variant, path=path, loaded=loaded))

    def costs(self, batch):
        return [self.wl.layer_costs(l["L"], batch, l["nnz"]) for l in self.layers]

    def settle_variants(self, batch, stream):
        """A forced variant that does not cover a layer (e.g. tensor cores with 6 input channels)
        falls back to the engine's own choice for that layer."""
        for l in self.layers:
            L = l["L"]
            try:
                self.tb.sparse_conv2d(l["f"], l["x"], l["y"], batch, L.H, L.W, L.stride, L.pad,
                                      cuda_stream=stream, variant=l["variant"])
            except self.tb.TetrisError as e:
                if e.status != 3:
                    raise
                l["variant"] = 0
        self.torch.cuda.synchronize()

    def tune(self, batch, stream):
        """Untimed set-up, as in the reference protocol (its tile search is not part of the
        timing, Tetris/spconv2d.cc:285-326): every layer times its best-ranked tile shapes and
        the tensor-core variant once for this batch and keeps the fastest."""
        if batch in self.tuned:
            return
        for l in self.layers:
            L = l["L"]
            if l["variant"] == 0 and not l["loaded"]:   # (a filter from the plan cache brings its tuned plans along)
                self.tb.tune_sparse_conv2d(l["f"], l["x"], l["y"], batch, L.H, L.W, L.stride, L.pad,
                                           cuda_stream=stream)
                if l["path"]:
                    l["f"].save(l["path"])
        self.tuned.add(batch)

    def kernels(self, batch):
        names = []
        for l in self.layers:
            L = l["L"]
            v = l["variant"] if l["variant"] != 0 else self.tb.auto_choice(l["f"], batch, L.H, L.W, L.stride, L.pad)
            names.append("depthwise" if L.groups != 1 else "generic" if v == 1 else
                         "%s_%dx%d_s%d" % (VARIANT_NAMES[v], L.KS, L.KS, L.stride))
        return names

    def launch_all(self, batch, stream, events=None, only=None):
        for i, l in enumerate(self.layers):
            if only is not None and i not in only:
                continue
            L = l["L"]
            self.tb.sparse_conv2d(l["f"], l["x"], l["y"], batch, L.H, L.W, L.stride, L.pad,
                                  cuda_stream=stream, variant=l["variant"])
            if events is not None:
                events[i + 1].record(stream)

    def check(self):
        for l in self.layers:
            l["f"].check()  # a tensor-core launch that gave up on a barrier is an error, not a result

    def time_graph(self, batch, steps, warmup, sync, only=None):
        """ms per step with the step's launches (or those of the layers in `only`) captured once
        and replayed as one CUDA graph (no per-launch host work; events around the K replays)."""
        torch = self.torch
        g = torch.cuda.CUDAGraph()
        self.launch_all(batch, torch.cuda.current_stream(), only=only)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            self.launch_all(batch, torch.cuda.current_stream(), only=only)
        for _ in range(warmup):
            g.replay()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            g.replay()
        e1.record()
        sync()
        self.check()
        return e0.elapsed_time(e1) / steps

    def parity(self, batch, orc):
        """The outputs the timed launches left behind, against the CPU oracle: images 0 and
        batch-1 of every layer on a 16-channel slice (the oracle on a slice of the filter is
        cheap; the device computed the whole layer)."""
        tot = {"layers": 0, "bad": 0, "max_abs": 0.0, "max_rel": 0.0, "n_floor": 0, "elements": 0}
        per_layer = []
        for idx, l in enumerate(self.layers):
            L = l["L"]
            imgs = sorted({0, batch - 1})
            oc0 = min(max(L.OC - 16, 0), (idx * 24) % max(L.OC, 1))
            oc1 = min(L.OC, oc0 + 16)
            xs = l["x"][imgs].permute(0, 3, 1, 2).contiguous().cpu().numpy()
            got = l["y"][imgs][..., oc0:oc1].permute(0, 3, 1, 2).contiguous().cpu().numpy()
            if L.groups != 1:
                want = orc.host_depthwise_conv2d(xs[:, oc0:oc1], l["filt"][oc0:oc1], L.stride, L.pad)
            else:
                want = orc.host_conv2d(xs, l["filt"][oc0:oc1], L.stride, L.pad, threads=True, skip_zero=True)
            bad, max_rel, n_floor = orc.compare(got, want)
            bad += int(np.isnan(got).sum())
            max_abs = float(np.abs(got - want).max())
            per_layer.append({"bad": bad, "max_abs": max_abs, "n_floor": n_floor})
            tot["layers"] += 1; tot["bad"] += bad; tot["n_floor"] += n_floor; tot["elements"] += int(got.size)
            tot["max_abs"] = max(tot["max_abs"], max_abs); tot["max_rel"] = max(tot["max_rel"], max_rel)
        tot["bar"] = ("|got - want| <= 1e-4*max(|got|,|want|) + 1e-5 against HostConv2d; images 0 and N-1, "
                      "16 output channels per layer; n_floor = elements that pass through the 1e-5 floor only")
        return tot, per_layer


def cpu_reference_step(wl, workload, threads):
    """One image through every layer on the host cores with the reference's CPU convolution
    (oracle/_ref when it was compiled, else the C port).  Returns (seconds, kind)."""
    orc = oracle_module()
    from concurrent.futures import ThreadPoolExecutor
    use_ref = orc.ref() is not None
    total = 0.0
    pool = ThreadPoolExecutor(max_workers=threads)
    for idx, L in enumerate(wl.WORKLOADS[workload]()):
        filt = np.ascontiguousarray(wl.make_filter(workload, idx, L))
        x = np.ascontiguousarray(wl.make_input(workload, idx, L, 1))
        oh, ow = wl.out_extent(L.H, L.KS, L.stride, L.pad), wl.out_extent(L.W, L.KS, L.stride, L.pad)
        out = np.empty((1, L.OC, oh, ow), np.float32)
        t0 = time.perf_counter()
        if L.groups != 1:
            orc.port().oracle_host_depthwise_conv2d(x.ctypes.data, filt.ctypes.data, out.ctypes.data,
                                                    1, L.H, L.W, L.IC, L.KS, L.stride, L.pad)
        elif use_ref:
            # HostConv2d is single-threaded; output-channel slices are independent, so each
            # worker calls it on its own slice of the filter and of the output (same arithmetic).
            per = -(-L.OC // threads)
            def work(o0):
                o1 = min(L.OC, o0 + per)
                orc.ref().ref_host_conv2d(x.ctypes.data, filt[o0:o1].ctypes.data, out[0, o0:o1].ctypes.data,
                                          1, L.H, L.W, L.IC, o1 - o0, L.KS, L.stride, L.pad)
            list(pool.map(work, range(0, L.OC, per)))
        else:
            os.environ.setdefault("OMP_NUM_THREADS", str(threads))
            orc.port().oracle_host_conv2d_mt(x.ctypes.data, filt.ctypes.data, out.ctypes.data, 1, L.H,
                                             L.W, L.IC, L.OC, L.KS, L.stride, L.pad, 0)
        total += time.perf_counter() - t0
    pool.shutdown()
    return total, ("reference" if use_ref else "port")


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    for _ in range(min(args.warmup, 1)):
        cpu_reference_step(wl, args.workload, threads)
    t_total, kind = 0.0, "port"
    for _ in range(args.steps):
        t, kind = cpu_reference_step(wl, args.workload, threads)
        t_total += t
    per_image = t_total / args.steps
    value = 1.0 / per_image
    sample = "1 image per step through all %d conv layers (CPU images/s does not depend on the batch)" \
        % len(wl.WORKLOADS[args.workload]())
    print(json.dumps({
        "impl": "reference", "metric": "images_per_s", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_image * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%s_b%d" % (args.workload, args.batch),
                   "note": "reference CPU direct convolution (HostConv2d) on the host cores; each step is a "
                           "bounded sample of the workload: one image through every layer"},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": threads, "kind": kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="vgg19")
    ap.add_argument("--batch", type=int, default=16,
                    help="images per GPU (weak scaling), or the global batch with --scaling strong")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="strong: --batch is one global batch cut into per-rank slices")
    ap.add_argument("--variant", type=int, default=0, help="0 auto, 1 generic, 2 tiled, 4 tensor")
    ap.add_argument("--oc-block", type=int, default=0, help="output channels per register block (0 = default)")
    ap.add_argument("--tile-ic", type=int, default=0, help="input channels per stage (0 = default)")
    ap.add_argument("--no-cudnn-context", action="store_true", help="skip the cuDNN dense FP32 context line")
    ap.add_argument("--no-tune", action="store_true", help="skip the untimed tile auto-tuning pass")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the check of the timed outputs against the CPU oracle")
    ap.add_argument("--no-arms", action="store_true", help="skip timing both kernels (list, tensor-core) per layer")
    ap.add_argument("--no-workloads", action="store_true", help="skip the per-model block of the other workloads")
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling block of a multi-GPU run")
    ap.add_argument("--sustained-s", type=float, default=2.0, help="seconds of the sustained loop (0 = skip)")
    ap.add_argument("--e2e-slots", type=int, default=4, choices=[1, 2, 3, 4],
                    help="pipeline slots (stream + workspace) the end-to-end path rotates over")
    ap.add_argument("--plan-cache", default=None,
                    help="directory of compressed-filter files: filters and their tuned tile plans are "
                         "saved there after tuning and loaded from there by the next run")
    ap.add_argument("--quick", action="store_true", help="only the timed region and the roofline (for profiling runs)")
    args = ap.parse_args()
    if args.quick:
        args.no_cudnn_context = args.no_cpu_baseline = args.no_e2e = args.no_arms = True
        args.no_workloads = args.no_strong = args.no_parity = True
        args.sustained_s = 0.0

    tb = load_package()
    import importlib
    wl = importlib.import_module("tetris_b200.workloads")
    if args.impl == "reference":
        run_reference_arm(args, wl)
        return

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert args.warmup >= 3, "at least 3 warm-up steps"
    if args.plan_cache:
        os.makedirs(args.plan_cache, exist_ok=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.scaling == "strong":
        _, batch = tb.batch_slice(args.batch, world, rank)
        global_batch = args.batch
    else:
        batch, global_batch = args.batch, args.batch * world
    stream = torch.cuda.current_stream()
    model = Model(tb, wl, torch, args.workload, max(batch, 1), local, args.oc_block, args.tile_ic, args.variant,
                  args.plan_cache)
    layers = model.layers
    model.settle_variants(batch, stream)
    if not args.no_tune:
        model.tune(batch, stream)
    kernels = model.kernels(batch)

    # ---- per-layer breakdown: eager launches, one event per layer ----
    for _ in range(args.warmup):
        model.launch_all(batch, stream)
    barrier()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(layers) + 1)]
          for _ in range(args.steps)]
    for s in range(args.steps):
        ev[s][0].record(stream)
        model.launch_all(batch, stream, ev[s])
    barrier()
    model.check()
    step_ms = [ev[s][0].elapsed_time(ev[s][-1]) for s in range(args.steps)]
    total_ms = ev[0][0].elapsed_time(ev[-1][-1])
    layer_ms = [float(np.mean([ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)]))
                for i in range(len(layers))]
    eager_ms_per_step = max_over_ranks(total_ms) / args.steps

    # ---- the timed outputs against the CPU oracle (the checker, not a compute path) ----
    parity = parity_layers = None
    if not args.no_parity and rank == 0:
        parity, parity_layers = model.parity(batch, oracle_module())

    # ---- THE TIMED REGION: the same step, its launches captured once and replayed K times as one
    #      CUDA graph (no per-launch host work between the layers of a step); barrier + synchronise
    #      on both sides, CUDA events on the launching stream, max over ranks.  The eager pass
    #      above gives the per-layer breakdown. ----
    launches_before = tb.launch_count()
    model.launch_all(batch, stream)
    launches_per_step = tb.launch_count() - launches_before
    sampler = ClockSampler(local).start() if rank == 0 else None
    ms_per_step = max_over_ranks(model.time_graph(batch, args.steps, args.warmup, barrier))
    clocks = sampler.stop() if rank == 0 else None
    value = global_batch / (ms_per_step * 1e-3)
    gpu_launches = launches_per_step * args.steps  # kernels of the library per replayed step x K steps
    eager_info = {"ms_per_step": eager_ms_per_step, "images_per_s": global_batch / (eager_ms_per_step * 1e-3),
                  "note": "the same K steps launched one by one from Python with an event per layer (per-layer breakdown)"}

    # ---- both kernels per layer (list kernel on the CUDA cores, dense contraction on the
    #      tensor cores), so that the automatic choice can be audited ----
    arms = None
    if not args.no_arms and world == 1:
        arms = []
        for l in layers:
            L = l["L"]
            rec = {}
            for name, v in (("tiled_ms", tb.VARIANT_TILED), ("tensor_ms", tb.VARIANT_TENSOR),
                            ("tensor16_ms", tb.VARIANT_TENSOR16)):
                try:
                    rec[name] = tb.timing_sparse_conv2d(l["f"], l["x"], l["y"], batch, L.H, L.W, L.stride, L.pad,
                                                        cuda_stream=stream, variant=v, warm=2, repeat=5) \
                        if L.groups == 1 else None
                except tb.TetrisError:
                    rec[name] = None
            arms.append(rec)

    # ---- real pruned layers beside their uniform-mask twins (same shape, same nonzero values at
    #      uniformly random positions): what the skew of magnitude-pruned rows costs each kernel ----
    skew = None
    if args.workload == "real" and world == 1:
        skew = []
        for l in layers:
            L = l["L"]
            twin = tb.SparseFilter(wl.uniform_like(l["filt"], seed=7), L.IC, L.OC, L.KS, device=local)
            rows = np.count_nonzero(l["filt"].reshape(L.OC, -1), axis=1)
            rec = {"name": L.name, "row_nnz_min_mean_max": [int(rows.min()), float(rows.mean()), int(rows.max())],
                   "empty_rows": int((rows == 0).sum())}
            for key, v in (("tiled", tb.VARIANT_TILED), ("auto", tb.VARIANT_AUTO)):
                if v == tb.VARIANT_AUTO:
                    tb.tune_sparse_conv2d(twin, l["x"], l["y"], batch, L.H, L.W, L.stride, L.pad, cuda_stream=stream)
                a = tb.timing_sparse_conv2d(l["f"], l["x"], l["y"], batch, L.H, L.W, L.stride, L.pad, variant=v, warm=3, repeat=10)
                b = tb.timing_sparse_conv2d(twin, l["x"], l["y"], batch, L.H, L.W, L.stride, L.pad, variant=v, warm=3, repeat=10)
                rec[key + "_real_ms"], rec[key + "_uniform_ms"], rec[key + "_skew_penalty"] = a, b, a / b - 1.0
            skew.append(rec)
            twin.close()

    # ---- sustained: the step looped for seconds, with the clocks and the power seen ----
    sustained = None
    if args.sustained_s > 0 and world == 1:
        reps = max(args.steps, int(args.sustained_s * 1e3 / ms_per_step) + 1)
        smp = ClockSampler(local).start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            model.launch_all(batch, stream)
        e1.record(stream)
        torch.cuda.synchronize()
        c = smp.stop()
        sms_ = e0.elapsed_time(e1) / reps
        sustained = {"steps": reps, "seconds": e0.elapsed_time(e1) * 1e-3, "ms_per_step": sms_,
                     "images_per_s": batch / (sms_ * 1e-3), "sm_mhz_median": c["sm_mhz"],
                     "power_w_median": c.get("power_w_median"), "power_w_max": c.get("power_w_max"),
                     "reasons": c["reasons"],
                     "ms_x_mhz": sms_ * c["sm_mhz"] if c["sm_mhz"] else None}

    # ---- end to end: host buffers in, host buffers out, through the host-pointer entry point ----
    e2e = None
    if not args.no_e2e:
        hin = [torch.empty(batch, l["L"].IC, l["L"].H, l["L"].W).pin_memory() for l in layers]
        hout = [torch.empty(batch, l["L"].OC, l["oh"], l["ow"]).pin_memory() for l in layers]
        for h, l in zip(hin, layers):
            h.copy_(l["x"][:batch].permute(0, 3, 1, 2))
        hin_np = [h.numpy() for h in hin]
        hout_np = [h.numpy() for h in hout]

        def e2e_step():
            # host buffers in, host buffers out; rotating pipeline slots, so the upload of one layer
            # overlaps the download of the previous ones; every result is on the host at the end
            for i, (h_in, h_out, l) in enumerate(zip(hin_np, hout_np, layers)):
                L = l["L"]
                tb.host_sync(local, i % args.e2e_slots)
                tb.cuda_sparse_conv2d_async(h_in, l["f"], batch, L.H, L.W, L.stride, L.pad,
                                            h_out, slot=i % args.e2e_slots)
            tb.host_sync(local, -1)
        e2e_steps = max(1, min(args.steps, 3))
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        te = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        h2d, d2h = int(sum(h.numel() * 4 for h in hin)), int(sum(h.numel() * 4 for h in hout))
        # what the host link gives this rank while all ranks copy at once: 256 MiB each way on two
        # streams.  When this figure falls as ranks are added, the platform (host memory, PCIe
        # root ports shared between GPUs), not the engine, is what limits e2e.
        probe = torch.empty(64 << 20).pin_memory()
        probe2 = torch.empty(64 << 20).pin_memory()
        dprobe, dprobe2 = torch.empty(64 << 20, device="cuda"), torch.empty(64 << 20, device="cuda")
        s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
        barrier()
        t0 = time.perf_counter()
        for _ in range(3):
            with torch.cuda.stream(s1):
                dprobe.copy_(probe, non_blocking=True)
            with torch.cuda.stream(s2):
                probe2.copy_(dprobe2, non_blocking=True)
        torch.cuda.synchronize()
        link = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": global_batch / te, "unit": "images/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "host_link_gbs_per_rank": 3 * 2 * (256 << 20) / link / 1e9,
               "copy_gbs_per_rank": (h2d + d2h) / te / 1e9,
               "note": "limited by the host link: copy_gbs_per_rank against host_link_gbs_per_rank (a plain "
                       "pinned-memory copy both ways, all ranks at once)"}
        del hin, hout, hin_np, hout_np, probe, probe2, dprobe, dprobe2

    # ---- strong scaling: one global batch cut into per-rank slices (the batch partitioner),
    #      step = CUDA-graph replay of the rank's slice, max over ranks; the same batch on one GPU
    #      is timed in the same run for the efficiency ----
    strong = None
    if world > 1 and not args.no_strong and args.scaling == "weak":
        strong = []
        for wname, gb in ((args.workload, 16), (args.workload, 64), ("yolov3", 16)):
            if gb < world:
                continue
            m = model if wname == args.workload and gb <= model.max_batch else \
                Model(tb, wl, torch, wname, gb, local, args.oc_block, args.tile_ic, args.variant)
            _, mine = tb.batch_slice(gb, world, rank)
            m.settle_variants(gb, stream)
            if not args.no_tune:
                m.tune(gb, stream); m.tune(mine, stream)
            t_all = max_over_ranks(m.time_graph(gb, max(5, args.steps // 4), 3, barrier))
            t_mine = max_over_ranks(m.time_graph(mine, max(5, args.steps // 2), 3, barrier))
            # which layers stop scaling: per-layer time of the slice over 1/world of the full batch
            worst = None
            if rank == 0:
                ratios = []
                for l in m.layers:
                    L = l["L"]
                    a = tb.timing_sparse_conv2d(l["f"], l["x"], l["y"], gb, L.H, L.W, L.stride, L.pad, warm=3, repeat=10)
                    b = tb.timing_sparse_conv2d(l["f"], l["x"], l["y"], mine, L.H, L.W, L.stride, L.pad, warm=3, repeat=10)
                    ratios.append((b * world / a, L.name, "%dx%d %d->%d %dx%d s%d" % (L.H, L.W, L.IC, L.OC, L.KS, L.KS, L.stride)))
                ratios.sort(reverse=True)
                worst = [{"layer": n, "shape": s, "slice_time_x_ranks_over_full_time": r} for r, n, s in ratios[:3]]
            strong.append({"workload": wname, "global_batch": gb, "images_per_gpu": mine,
                           "ms_per_step": t_mine, "images_per_s": gb / (t_mine * 1e-3),
                           "one_gpu_ms_per_step": t_all, "efficiency_vs_n1": t_all / (world * t_mine),
                           "layers_that_scale_worst": worst})
            if m is not model:
                del m
                torch.cuda.empty_cache()

    # ---- one call cut over the GPUs of this box from ONE process (tetris_conv2d_host_sharded), one
    #      filter per distinct device, against the single-GPU result ----
    sharded = None
    if world > 1 and rank == 0:
        L = wl.WORKLOADS["single"]()[0]
        filt = wl.make_filter("single", 0, L)
        xs = wl.make_input("single", 0, L, 16)
        ndev = min(world, torch.cuda.device_count())
        fs = [tb.SparseFilter(filt, L.IC, L.OC, L.KS, device=d) for d in range(ndev)]
        one = tb.cuda_sparse_conv2d(xs, fs[local], 16, L.H, L.W, L.stride, L.pad)
        cut = tb.cuda_sparse_conv2d_sharded(xs, fs, 16, L.H, L.W, L.stride, L.pad)
        sharded = {"gpus": ndev, "batch": 16, "identical_to_one_gpu": bool(np.array_equal(one, cut)),
                   "max_abs_diff": float(np.abs(one - cut).max())}
        for f in fs:
            f.close()
    barrier()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    hbm_gbs, peak_src = read_peaks()
    sms, khz, lanes = tb.device_info(local)
    fp32_peak = sms * lanes * 2 * khz * 1e3  # FLOP/s

    def roof_s(costs):
        return sum(max(b / (hbm_gbs * 1e9), f / fp32_peak) for f, b in costs)

    # ---- per-model figures of the other workloads (batch 16, and batch 1), each after tuning:
    #      Sigma-layer latency as a CUDA-graph replay and as the sum of the per-layer means of the
    #      reference's timing protocol, against the Sigma-layer roofline ----
    workloads_block = None
    if not args.no_workloads and world == 1:
        workloads_block = []
        for wname, batches in (("single", (1,)), ("vgg19", (1,)), ("resnet50", (16, 1)), ("mobilenet", (16, 1)),
                               ("yolov3", (16,))):
            m = Model(tb, wl, torch, wname, max(batches), local)
            for b in batches:
                m.settle_variants(b, stream)
                m.tune(b, stream)
                t_layers = sum(tb.timing_sparse_conv2d(l["f"], l["x"], l["y"], b, l["L"].H, l["L"].W, l["L"].stride,
                                                       l["L"].pad, warm=5, repeat=20) for l in m.layers)
                t_graph = m.time_graph(b, 20, 3, torch.cuda.synchronize)
                pt = None if args.no_parity else m.parity(b, oracle_module())[0]
                workloads_block.append({
                    "workload": "%s_b%d" % (wname, b), "layers": len(m.layers),
                    "ms_per_step_graph": t_graph, "images_per_s": b / (t_graph * 1e-3),
                    "sum_layer_ms": t_layers, "roofline_frac": roof_s(m.costs(b)) / (t_graph * 1e-3),
                    "roofline_frac_sum_layers": roof_s(m.costs(b)) / (t_layers * 1e-3),
                    "parity_bad": pt["bad"] if pt else None, "parity_max_abs": pt["max_abs"] if pt else None})
            del m
            torch.cuda.empty_cache()

    # ---- context line: cuDNN dense FP32 convolution (a library, not this engine) on the same
    #      shapes, as the reference does with CuDNNConv2d (Tetris/cuda_utils.cc:6-132: the fastest
    #      algorithm cuDNN finds per shape, 30 warm-up + 100 timed launches per layer) ----
    cudnn = None
    if world == 1 and not args.no_cudnn_context:
        import torch.nn.functional as F
        torch.backends.cudnn.benchmark = True          # cuDNN times its algorithms per shape and keeps the fastest
        torch.backends.cudnn.allow_tf32 = False        # FP32 arithmetic, like the engine
        torch.backends.cuda.matmul.allow_tf32 = False
        cms_layers = []
        for l in layers:
            L = l["L"]
            w = torch.from_numpy(l["filt"]).cuda().contiguous(memory_format=torch.channels_last)
            x = l["x"][:batch].permute(0, 3, 1, 2)     # NHWC storage seen as NCHW channels_last
            for _ in range(tb.WARM):
                F.conv2d(x, w, None, L.stride, L.pad, 1, L.groups)
            torch.cuda.synchronize()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record()
            for _ in range(tb.REPEAT):
                F.conv2d(x, w, None, L.stride, L.pad, 1, L.groups)
            c1.record()
            torch.cuda.synchronize()
            cms_layers.append(c0.elapsed_time(c1) / tb.REPEAT)
        cms = float(sum(cms_layers))
        cudnn = {"ms_per_step": cms, "images_per_s": batch / (cms * 1e-3), "dtype": "f32 (TF32 off)",
                 "layout": "channels_last", "protocol": "per layer: 30 warm-up + 100 timed launches, summed",
                 "note": "dense convolution by cuDNN through torch (fastest algorithm per shape); context, not a target"}

    # ---- roofline of the dominant kernel ----
    costs = model.costs(batch)
    per_layer = []
    for i, (l, ms, kind, (flops, nbytes)) in enumerate(zip(layers, layer_ms, kernels, costs)):
        L = l["L"]
        t_roof = max(nbytes / (hbm_gbs * 1e9), flops / fp32_peak)
        rec = {"name": L.name, "kernel": kind, "ms": ms, "nnz": l["nnz"],
               "gbs": nbytes / (ms * 1e-3) / 1e9, "tflops": flops / (ms * 1e-3) / 1e12,
               "bound": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / fp32_peak else "fp32",
               "roofline_frac": t_roof / (ms * 1e-3)}
        if arms:
            rec.update(arms[i])
        if parity_layers:
            rec["parity_max_abs"] = parity_layers[i]["max_abs"]
            rec["parity_n_floor"] = parity_layers[i]["n_floor"]
        per_layer.append(rec)
    by_kernel = {}
    for pl, (flops, nbytes) in zip(per_layer, costs):
        k = by_kernel.setdefault(pl["kernel"], {"ms": 0.0, "flops": 0, "bytes": 0, "launches": 0})
        k["ms"] += pl["ms"]; k["flops"] += flops; k["bytes"] += nbytes; k["launches"] += 1
    top = max(by_kernel, key=lambda k: by_kernel[k]["ms"])
    tk = by_kernel[top]
    # the dominant kernel's launches alone, replayed like the timed region (CUDA events around K replays)
    top_layers = {i for i, pl in enumerate(per_layer) if pl["kernel"] == top}
    tk["eager_ms"] = tk["ms"]
    tk["ms"] = model.time_graph(batch, args.steps, args.warmup, torch.cuda.synchronize, only=top_layers)
    t_hbm = tk["bytes"] / (hbm_gbs * 1e9)
    t_fp = tk["flops"] / fp32_peak
    if t_hbm >= t_fp:
        roofline = {"bound": "hbm", "achieved": tk["bytes"] / (tk["ms"] * 1e-3) / 1e9, "peak": hbm_gbs,
                    "unit": "GB/s"}
    else:
        roofline = {"bound": "fp32", "achieved": tk["flops"] / (tk["ms"] * 1e-3) / 1e12,
                    "peak": fp32_peak / 1e12, "unit": "TFLOP/s"}
    roofline["frac"] = roofline["achieved"] / roofline["peak"]
    roofline.update({
        "kernel": top, "launches_per_step": tk["launches"],
        "traffic": NCU_TRAFFIC[top]["dram_over_algorithmic"] * tk["bytes"] / tk["launches"]
                   if top in NCU_TRAFFIC else None,
        "traffic_note": NCU_TRAFFIC[top]["note"] if top in NCU_TRAFFIC else None,
        "peak_source": ("%s HBM copy bandwidth; FP32 peak = %d SMs x %d lanes x 2 x %.0f MHz"
                        % (peak_src, sms, lanes, khz / 1e3)),
        "hbm_gbs_achieved": tk["bytes"] / (tk["ms"] * 1e-3) / 1e9, "hbm_gbs_peak": hbm_gbs,
        "algorithmic_bytes_per_step": tk["bytes"], "nonzero_flops_per_step": tk["flops"],
        "share_of_step_time": tk["ms"] / ms_per_step,
        "ms_per_step_of_this_kernel": tk["ms"], "ms_per_step_of_this_kernel_eager": tk["eager_ms"],
    })

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:  # the CPU baseline is a single-GPU-run extra
        threads = os.cpu_count() or 1
        secs, kind = cpu_reference_step(wl, args.workload, threads)
        cpu_baseline = {"value": 1.0 / secs, "unit": "images/s", "cores": threads, "kind": kind,
                        "sample": "1 image through all %d conv layers, once (%.1f s)" % (len(layers), secs)}

    top_family = top.split("_")[0]
    print(json.dumps({
        "metric": "images_per_s", "value": value, "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "arith": ARITH.get(top_family, "FP32"),
        "data": "synthetic",
        "config": {"workload": "%s_b%d" % (args.workload, args.batch), "batch_per_gpu": batch,
                   "global_batch": global_batch, "layers": len(layers), "variant": args.variant,
                   "l2": "a step touches %.0f MB of activations, more than the 126 MB L2, before a "
                         "layer runs again" % (sum(b for _, b in costs) / 1e6)},
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": int(gpu_launches), "clocks": clocks, "parity": parity,
        "model_roofline_frac": roof_s(costs) / (ms_per_step * 1e-3),
        "layers_at_half_roofline": sum(1 for p in per_layer if p["roofline_frac"] >= 0.5),
        "step_ms_min_max": [min(step_ms), max(step_ms)],
        "timed_as": "CUDA-graph replay of the step's launches", "eager": eager_info, "sustained": sustained, "strong": strong, "sharded_one_process": sharded,
        "cudnn_context": cudnn, "cudnn_ms_per_step": cudnn["ms_per_step"] if cudnn else None,
        "workloads": workloads_block, "real_vs_uniform": skew,
        "per_layer": per_layer,
    }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
