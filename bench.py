"""Benchmark of the sparse-filter convolution path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload vgg19] [--batch 16]
    python bench.py --impl reference ...        # the reference's CPU path on the host cores

A step is one pass over one batch: every conv layer of the workload launched back to back, each
on its own synthetic input that already sits in HBM.  The metric is whole-job images/s (batch *
ranks / step time); ms_per_step is the per-model sum-of-layers sparse-conv latency the
reference reports (evalution/overall_speedup.py:159-165).  One JSON line goes to stdout.

Multi-GPU: one process per GPU (torchrun); each rank runs the same per-GPU batch on its own
device (independent batch shards, no collective on the data path), the step time is the max over
ranks.
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
    "tensor_3x3_s1": {"dram_over_algorithmic": 65.7 / 107.5,
                      "note": "captured on VGG-19 conv3_3 batch 16: 65.7 MB per launch against 107.5 MB "
                              "algorithmic (outputs still in L2 at kernel end); scaled by algorithmic bytes"},
    "tiled_3x3_s1": {"dram_over_algorithmic": 270.5 / 205.7,
                     "note": "captured on VGG-19 conv2_2 batch 16: 270.5 MB per launch against 205.7 MB "
                             "algorithmic; scaled by algorithmic bytes"},
}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
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

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_layers(tb, wl, workload, batch, torch, device, oc_block=0, tile_ic=0):
    """Compress every layer's filter on the device and allocate its NHWC input and output."""
    layers = []
    for idx, L in enumerate(wl.WORKLOADS[workload]()):
        filt = wl.make_filter(workload, idx, L)
        f = tb.SparseFilter(filt, L.IC, L.OC, L.KS, TILE_IC=tile_ic, groups=L.groups, device=device,
                            oc_block=oc_block)
        oh, ow = wl.out_extent(L.H, L.KS, L.stride, L.pad), wl.out_extent(L.W, L.KS, L.stride, L.pad)
        g = torch.Generator(device="cuda").manual_seed(1000 + idx)
        x = torch.rand(batch, L.H, L.W, L.IC, device="cuda", generator=g)
        x = x * (torch.rand(x.shape, device="cuda", generator=g) >= 0.5)
        y = torch.empty(batch, oh, ow, L.OC, device="cuda")
        flops, nbytes = wl.layer_costs(L, batch, int(f.nnz_))
        layers.append(dict(L=L, f=f, x=x, y=y, oh=oh, ow=ow, flops=flops, bytes=nbytes,
                           nnz=int(f.nnz_), filt=filt))
    return layers


def cpu_reference_step(wl, workload, threads):
    """One image through every layer on the host cores with the reference's CPU convolution
    (oracle/_ref when it was compiled, else the C port).  Returns (seconds, kind)."""
    from oracle import oracle as orc
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
                   "note": "reference CPU direct convolution (HostConv2d) on the host cores"},
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
    ap.add_argument("--batch", type=int, default=16, help="images per GPU")
    ap.add_argument("--variant", type=int, default=0, help="0 auto, 1 generic, 2 tiled")
    ap.add_argument("--oc-block", type=int, default=0, help="output channels per register block (0 = default)")
    ap.add_argument("--tile-ic", type=int, default=0, help="input channels per stage (0 = default)")
    ap.add_argument("--cudnn-context", action="store_true",
                    help="(kept for old command lines: the cuDNN context line is on by default at one GPU)")
    ap.add_argument("--no-cudnn-context", action="store_true",
                    help="skip the cuDNN dense FP32 context line")
    ap.add_argument("--no-tune", action="store_true", help="skip the untimed tile auto-tuning pass")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-slots", type=int, default=4, choices=[1, 2, 3, 4],
                    help="pipeline slots (stream + workspace) the end-to-end path rotates over")
    ap.add_argument("--graph", action="store_true",
                    help="also time the step replayed as one CUDA graph (reported as `cuda_graph`)")
    args = ap.parse_args()

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
        os.environ["NCCL_DEBUG"] = "WARN"  # NCCL's version banner would land on stdout beside the JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert args.warmup >= 3, "at least 3 warm-up steps"

    layers = build_layers(tb, wl, args.workload, args.batch, torch, local, args.oc_block, args.tile_ic)
    stream = torch.cuda.current_stream()

    # a forced variant that does not cover a layer (e.g. tensor cores with 3 input channels)
    # falls back to the engine's own choice for that layer
    for l in layers:
        L = l["L"]
        l["variant"] = args.variant
        try:
            tb.sparse_conv2d(l["f"], l["x"], l["y"], args.batch, L.H, L.W, L.stride, L.pad,
                             cuda_stream=stream, variant=args.variant)
        except tb.TetrisError as e:
            if e.status != 3:
                raise
            l["variant"] = 0
    torch.cuda.synchronize()

    def launch_all(events=None, st=None):
        st = st or stream
        for i, l in enumerate(layers):
            L = l["L"]
            tb.sparse_conv2d(l["f"], l["x"], l["y"], args.batch, L.H, L.W, L.stride, L.pad,
                             cuda_stream=st, variant=l["variant"])
            if events is not None:
                events[i + 1].record(st)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Untimed set-up, as in the reference protocol (its tile search is not part of the timing,
    # Tetris/spconv2d.cc:285-326): let every layer time its best-ranked tile shapes once.
    if not args.no_tune and args.variant == 0:
        for l in layers:
            L = l["L"]
            tb.tune_sparse_conv2d(l["f"], l["x"], l["y"], args.batch, L.H, L.W, L.stride, L.pad,
                                  cuda_stream=stream)

    # what the engine's automatic choice is per layer, for the report (after the tuning pass)
    for l in layers:
        L = l["L"]
        l["kernel_variant"] = l["variant"] if l["variant"] != 0 else \
            tb.auto_choice(l["f"], args.batch, L.H, L.W, L.stride, L.pad)

    # ---- device-resident throughput ----
    for _ in range(args.warmup):
        launch_all()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(layers) + 1)]
          for _ in range(args.steps)]
    for s in range(args.steps):
        ev[s][0].record(stream)
        launch_all(ev[s])
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    for l in layers:
        l["f"].check()  # a tensor-core launch that gave up on a barrier is an error, not a result
    step_ms = [ev[s][0].elapsed_time(ev[s][-1]) for s in range(args.steps)]
    total_ms = ev[0][0].elapsed_time(ev[-1][-1])
    layer_ms = [float(np.mean([ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)]))
                for i in range(len(layers))]
    t = torch.tensor([total_ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps

    # ---- the same step as one CUDA graph (all layer launches captured once, replayed): what a
    #      layer chain costs without the per-launch host work; an extra figure, not `value` ----
    graph_info = None
    if args.graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            launch_all(st=torch.cuda.current_stream())
        for _ in range(args.warmup):
            g.replay()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            g.replay()
        g1.record()
        barrier()
        for l in layers:
            l["f"].check()
        tg = torch.tensor([g0.elapsed_time(g1)], device="cuda")
        if world > 1:
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        gms = float(tg.item()) / args.steps
        graph_info = {"ms_per_step": gms, "images_per_s": args.batch * world / (gms * 1e-3)}
    value = args.batch * world / (ms_per_step * 1e-3)

    # ---- end to end: host buffers in, host buffers out, through the host-pointer entry point ----
    e2e = None
    if not args.no_e2e:
        hin = [torch.empty(args.batch, l["L"].IC, l["L"].H, l["L"].W).pin_memory() for l in layers]
        hout = [torch.empty(args.batch, l["L"].OC, l["oh"], l["ow"]).pin_memory() for l in layers]
        for h, l in zip(hin, layers):
            h.copy_(l["x"].permute(0, 3, 1, 2))

        hin_np = [h.numpy() for h in hin]
        hout_np = [h.numpy() for h in hout]

        def e2e_step():
            # host buffers in, host buffers out; rotating pipeline slots, so the upload of one layer
            # overlaps the download of the previous ones; every result is on the host at the end
            for i, (h_in, h_out, l) in enumerate(zip(hin_np, hout_np, layers)):
                L = l["L"]
                tb.host_sync(local, i % args.e2e_slots)
                tb.cuda_sparse_conv2d_async(h_in, l["f"], args.batch, L.H, L.W, L.stride, L.pad,
                                            h_out, slot=i % args.e2e_slots)
            tb.host_sync(local, -1)
        e2e_steps = max(1, min(args.steps, 3))
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        te = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device="cuda")
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = {"value": args.batch * world / float(te.item()), "unit": "images/s",
               "h2d_bytes_per_step": int(sum(h.numel() * 4 for h in hin)),
               "d2h_bytes_per_step": int(sum(h.numel() * 4 for h in hout)),
               "steps": e2e_steps}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- context line: cuDNN dense FP32 convolution (a library, not this engine) on the same
    #      shapes, as the reference does with CuDNNConv2d (Tetris/cuda_utils.cc:6-132) ----
    cudnn = None
    if (args.cudnn_context or world == 1) and not args.no_cudnn_context:
        import torch.nn.functional as F
        torch.backends.cudnn.benchmark = True          # cuDNN picks its fastest algorithm per shape
        torch.backends.cudnn.allow_tf32 = False        # FP32 arithmetic, like the engine
        torch.backends.cuda.matmul.allow_tf32 = False
        dense = []
        for l in layers:
            L = l["L"]
            w = torch.from_numpy(l["filt"]).cuda().contiguous(memory_format=torch.channels_last)
            x = l["x"].permute(0, 3, 1, 2)             # NHWC storage seen as NCHW channels_last
            dense.append((x, w, L))
        def cudnn_step():
            for x, w, L in dense:
                F.conv2d(x, w, None, L.stride, L.pad, 1, L.groups)
        for _ in range(3):
            cudnn_step()
        torch.cuda.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, min(args.steps, 10))
        c0.record()
        for _ in range(reps):
            cudnn_step()
        c1.record()
        torch.cuda.synchronize()
        cms = c0.elapsed_time(c1) / reps
        cudnn = {"ms_per_step": cms, "images_per_s": args.batch / (cms * 1e-3), "dtype": "f32 (TF32 off)",
                 "layout": "channels_last", "note": "dense convolution by cuDNN through torch; context, not a target"}

    # ---- roofline of the dominant kernel ----
    hbm_gbs, peak_src = read_peaks()
    sms, khz, lanes = tb.device_info(local)
    fp32_peak = sms * lanes * 2 * khz * 1e3  # FLOP/s
    per_layer = []
    for l, ms in zip(layers, layer_ms):
        L = l["L"]
        names = {0: "tiled", 1: "generic", 2: "tiled", 4: "tensor"}
        kind = "depthwise" if L.groups != 1 else (
            "generic" if l["kernel_variant"] == 1 else
            "%s_%dx%d_s%d" % (names[l["kernel_variant"]], L.KS, L.KS, L.stride))
        t_roof = max(l["bytes"] / (hbm_gbs * 1e9), l["flops"] / fp32_peak)
        per_layer.append({"name": L.name, "kernel": kind, "ms": ms, "nnz": l["nnz"],
                          "gbs": l["bytes"] / (ms * 1e-3) / 1e9,
                          "tflops": l["flops"] / (ms * 1e-3) / 1e12,
                          "roofline_frac": t_roof / (ms * 1e-3)})
    by_kernel = {}
    for pl, l in zip(per_layer, layers):
        k = by_kernel.setdefault(pl["kernel"], {"ms": 0.0, "flops": 0, "bytes": 0, "launches": 0})
        k["ms"] += pl["ms"]; k["flops"] += l["flops"]; k["bytes"] += l["bytes"]; k["launches"] += 1
    top = max(by_kernel, key=lambda k: by_kernel[k]["ms"])
    tk = by_kernel[top]
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
        "share_of_step_time": tk["ms"] / sum(layer_ms),
    })

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:  # the CPU baseline is a single-GPU-run extra
        threads = os.cpu_count() or 1
        secs, kind = cpu_reference_step(wl, args.workload, threads)
        cpu_baseline = {"value": 1.0 / secs, "unit": "images/s", "cores": threads, "kind": kind,
                        "sample": "1 image through all %d conv layers, once (%.1f s)" % (len(layers), secs)}

    t_roof_sum = sum(max(l["bytes"] / (hbm_gbs * 1e9), l["flops"] / fp32_peak) for l in layers)
    print(json.dumps({
        "metric": "images_per_s", "value": value, "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "%s_b%d" % (args.workload, args.batch), "batch_per_gpu": args.batch,
                   "layers": len(layers), "variant": args.variant,
                   "l2": "a step touches %.0f MB of activations, more than the 126 MB L2, before a "
                         "layer runs again" % (sum(l["bytes"] for l in layers) / 1e6)},
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": args.steps * len(layers), "clocks": clocks,
        "model_roofline_frac": t_roof_sum / (sum(layer_ms) * 1e-3),
        "step_ms_min_max": [min(step_ms), max(step_ms)],
        "cudnn_context": cudnn, "cuda_graph": graph_info,
        "per_layer": per_layer,
    }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
