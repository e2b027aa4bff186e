"""Per-layer driver with the reference program's contract (Tetris/spconv2d.cc:369-450).

    python tetris-artifact-evalution_b200/spconv2d_test.py <weight_file> [batch]
    python tetris-artifact-evalution_b200/spconv2d_test.py --synthetic vgg19:5 [batch]

<weight_file> is a layer dump in the reference's text format: header `H W IC OC KS Pad S G`,
then OC*IC*KS*KS floats in OIHW order (Tetris/tensor_utils.cc:66-78).  Prints the lines the
reference's Python driver scrapes (evalution/conv2d_timing.py:51-65):

    [Config] sparsity = ..., nnz = ..., batch_size = ..., ...
    Time of Spconv2d :<ms>ms
    FLOPS of Spconv2d :<dense-equivalent binary TFLOP/s>T

followed by one JSON line with the bytes, nonzero FLOP/s and roofline figures.  Timing is the
reference protocol: 30 warm-up launches, then the mean of 100 back-to-back launches.
With --check the result is compared with the CPU convolution and `Sparse Pass.` /
`Sparse Error.` is printed as the reference does when its BENCHMARK macro is off.
"""
import argparse
import importlib
import importlib.util
import json
import os
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


def _package():
    if "tetris_b200" in sys.modules:
        return sys.modules["tetris_b200"]
    spec = importlib.util.spec_from_file_location(
        "tetris_b200", os.path.join(_HERE, "__init__.py"), submodule_search_locations=[_HERE])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["tetris_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def read_config_and_data_from_file(path):
    """ReadConfigAndDataFromFile (Tetris/tensor_utils.cc:55-82): (Layer fields, dense OIHW)."""
    try:
        with open(path) as fh:
            tokens = fh.read().split()
    except OSError:
        print("Open file error.")
        sys.exit(1)
    h, w, ic, oc, ks, pad, stride, groups = (int(t) for t in tokens[:8])
    n = oc * ic * ks * ks
    filt = np.array(tokens[8:8 + n], dtype=np.float32).reshape(oc, ic, ks, ks)
    return (h, w, ic, oc, ks, pad, stride, groups), filt


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("weight_file", nargs="?")
    ap.add_argument("batch", nargs="?", type=int, default=4)  # the reference's default batch
    ap.add_argument("--synthetic", help="workload:layer_index, e.g. vgg19:5")
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--warm", type=int, default=None)
    ap.add_argument("--repeat", type=int, default=None)
    ap.add_argument("--tile-ic", type=int, default=0)
    ap.add_argument("--oc-block", type=int, default=0)
    ap.add_argument("--no-tune", action="store_true")
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args(argv)
    print("args : %d %s\n" % (len(sys.argv), " ".join(sys.argv)))

    tb = _package()
    wl = importlib.import_module("tetris_b200.workloads")
    import torch
    assert torch.cuda.is_available(), "no CUDA device: this program has no CPU path"
    torch.cuda.set_device(0)
    prop = torch.cuda.get_device_properties(0)
    print('GPU Device 0: "%s" with compute capability %d.%d\n' % (prop.name, prop.major, prop.minor))

    batch = args.batch
    if args.synthetic:
        name, idx = args.synthetic.split(":")
        L = wl.WORKLOADS[name]()[int(idx)]
        filt = wl.make_filter(name, int(idx), L)
        h, w, ic, oc, ks, pad, stride, groups = L.H, L.W, L.IC, L.OC, L.KS, L.pad, L.stride, L.groups
        x = wl.make_input(name, int(idx), L, batch)
    else:
        (h, w, ic, oc, ks, pad, stride, groups), filt = read_config_and_data_from_file(
            args.weight_file or "./conv_weight_data/vgg19/vgg19-92-acc-71.7/"
            "module8_0_module2_0_conv2d_3_H_56_W_56_IC_256_OC_256_KS_3_Pad_1_S_1_G_1")
        groups = 1  # the reference reads the field and ignores it
        x = np.random.default_rng(0).uniform(-1, 1, (batch, ic, h, w)).astype(np.float32)
    nnz = int(np.count_nonzero(filt))
    # PrintConv2dConfig, Tetris/tensor_utils.cc:43-53
    print("[Config] sparsity = %g, nnz = %d, batch_size = %d, img_h = %d, img_w = %d, in_channel = %d, "
          "out_channel = %d, kernel_size = %d, padding = %d, stride = %d\n"
          % (1.0 - nnz / filt.size, nnz, batch, h, w, ic, oc, ks, pad, stride))

    f = tb.SparseFilter(filt, ic, oc, ks, TILE_IC=args.tile_ic, groups=groups, oc_block=args.oc_block)
    oh, ow = tb.out_extent(h, ks, stride, pad), tb.out_extent(w, ks, stride, pad)
    xin = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    out = torch.empty(batch, oh, ow, oc, device="cuda")
    if not args.no_tune and args.variant in (0, 2):  # the reference times its best tile config
        tb.tune_sparse_conv2d(f, xin, out, batch, h, w, stride, pad, cuda_stream=torch.cuda.current_stream())
    ms = tb.timing_sparse_conv2d(f, xin, out, batch, h, w, stride, pad,
                                 cuda_stream=torch.cuda.current_stream(), variant=args.variant,
                                 warm=tb.WARM if args.warm is None else args.warm,
                                 repeat=tb.REPEAT if args.repeat is None else args.repeat)
    dense_flops = 2.0 * oh * ow * batch * oc * (1 if groups != 1 else ic) * ks * ks
    print("Time of Spconv2d :%gms" % ms)
    print("FLOPS of Spconv2d :%gT" % (dense_flops * 1000 / ms / 1024 ** 4))  # Tetris/spconv2d.cc:358

    L = wl.Layer("layer", h, w, ic, oc, ks, pad, stride, groups, None)
    flops, nbytes = wl.layer_costs(L, batch, nnz)
    sms, khz, lanes = tb.device_info(0)
    fp32_peak = sms * lanes * 2 * khz * 1e3
    print(json.dumps({"ms": ms, "nnz": nnz, "bytes": nbytes, "nonzero_flops": flops,
                      "gbs": nbytes / ms / 1e6, "nonzero_tflops": flops / ms / 1e9,
                      "fp32_peak_tflops": fp32_peak / 1e12,
                      "fp32_frac": flops / (ms * 1e-3) / fp32_peak}))
    if args.check:
        sys.path.insert(0, os.path.dirname(_HERE))
        from oracle import oracle as orc
        print("HostConv2d begin")
        want = (orc.host_depthwise_conv2d(x, filt, stride, pad) if groups != 1
                else orc.host_conv2d(x, filt, stride, pad))
        print("HostConv2d end")
        got = out.cpu().numpy().transpose(0, 3, 1, 2)
        bad, max_rel, _ = orc.compare(got, want)
        print("Sparse Pass." if bad == 0 else "Sparse Error.", "max rel err %.3g" % max_rel)


if __name__ == "__main__":
    main()
