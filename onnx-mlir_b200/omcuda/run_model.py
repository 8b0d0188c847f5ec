"""Run, time and verify a compiled model from the command line.

    python -m omcuda.run_model --load-model DIR [-o NAME] [options]

The options, the seed (42), the warm-up / iteration protocol and the printed
statistics follow onnx-mlir's utils/RunONNXModel.py (:128-360 arguments,
:1083-1165 protocol) for the part that deals with an already compiled model:

  --load-model DIR        folder that holds NAME.so and NAME.constants.bin
  -o, --default-model-name NAME   (default: model)
  --print-signatures, --print-input, --print-output
  --shape-info 0:2x128x768,1:...  shapes of inputs with dynamic dimensions
  --lower-bound / --upper-bound   float32:-1,uint8:0 ... range of random inputs
  --seed N                seed of the random inputs (default 42)
  -w, --warmup N          untimed runs;  -n, --n-iteration N  timed runs
  --save-ref DIR          save inputs and outputs (input_<i>.npy, output_<i>.npy:
                          numpy files, the onnx package that the reference's
                          protobuf files need is not a dependency here)
  --load-ref DIR          take inputs (and, with --verify=ref, expected outputs)
                          from such a folder
  --verify ref            compare the outputs with the reference outputs
  --verify-every-value    elementwise check with --rtol / --atol (defaults 0.05 /
                          0.01, the reference's)
  --device-resident       not in the reference: upload the inputs once and pass
                          device tensors, so the timed runs hold no PCIe copies
"""
import argparse
import os
import sys
import time

import numpy as np


def ordinal(n):
    suffix = "th" if 10 <= n % 100 <= 20 else {1: "st", 2: "nd", 3: "rd"}.get(n % 10, "th")
    return str(n) + suffix


def data_without_top_bottom_quartile(data, percent):
    data = np.sort(np.asarray(data))
    trim = int(percent * len(data) / 100)
    return data[trim:len(data) - trim] if len(data) - 2 * trim > 0 else data


def parse_bounds(text):
    out = {}
    for item in (text or "").split(","):
        if item:
            k, v = item.split(":")
            out[np.dtype(k)] = float(v)
    return out


def make_inputs(sigs, args):
    shapes = {}
    for item in (args.shape_info or "").split(","):
        if item:
            i, dims = item.split(":")
            shapes[int(i)] = [int(d) for d in dims.split("x")]
    lo, hi = parse_bounds(args.lower_bound), parse_bounds(args.upper_bound)
    rng = np.random.default_rng(int(args.seed))
    inputs = []
    for i, (dt, dims, name) in enumerate(sigs):
        shape = shapes.get(i, dims)
        if any(d < 0 for d in shape):
            sys.exit("input %d (%s) has dynamic dimensions %s: give --shape-info %d:AxBx..."
                     % (i, name, dims, i))
        if dt.kind == "f":
            a, b = lo.get(dt, -1.0), hi.get(dt, 1.0)
            inputs.append(rng.uniform(a, b, size=shape).astype(dt))
        else:
            info = np.iinfo(dt)
            a, b = int(lo.get(dt, info.min)), int(hi.get(dt, info.max))
            inputs.append(rng.integers(a, b + 1, size=shape).astype(dt))
    return inputs


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--load-model", metavar="PATH", required=True)
    ap.add_argument("-o", "--default-model-name", metavar="MODEL_NAME", default="model")
    ap.add_argument("--print-signatures", action="store_true")
    ap.add_argument("--print-input", action="store_true")
    ap.add_argument("--print-output", action="store_true")
    ap.add_argument("--shape-info", type=str)
    ap.add_argument("--lower-bound", type=str)
    ap.add_argument("--upper-bound", type=str)
    ap.add_argument("--seed", type=str, default="42")
    ap.add_argument("-w", "--warmup", type=int, default=0)
    ap.add_argument("-n", "--n-iteration", type=int, default=1)
    ap.add_argument("--save-ref", metavar="PATH")
    ap.add_argument("--load-ref", metavar="PATH")
    ap.add_argument("--verify", choices=["ref"])
    ap.add_argument("--verify-every-value", action="store_true")
    ap.add_argument("--rtol", type=str, default="0.05")
    ap.add_argument("--atol", type=str, default="0.01")
    ap.add_argument("--device-resident", action="store_true")
    args = ap.parse_args(argv)
    if args.verify and not args.verify_every_value:
        sys.exit("--verify needs --verify-every-value")
    if args.verify == "ref" and not args.load_ref:
        sys.exit("--verify=ref needs --load-ref")

    import omcuda
    from omcuda.session import OMExecutionSession, parse_signature
    so = os.path.join(args.load_model, args.default_model_name + ".so")
    print("Loading the compiled model ...")
    t0 = time.perf_counter()
    sess = OMExecutionSession(so)
    print("  took ", time.perf_counter() - t0, " seconds.\n")
    in_sig, out_sig = sess.input_signature(), sess.output_signature()
    if args.print_signatures:
        print("Model's input signature: ", in_sig.strip())
        print("Model's output signature: ", out_sig.strip())
    sigs = parse_signature(in_sig)

    ref_outs = None
    if args.load_ref:
        inputs = [np.load(os.path.join(args.load_ref, "input_%d.npy" % i))
                  for i in range(len(sigs))]
        if args.verify == "ref":
            n_out = len(parse_signature(out_sig))
            ref_outs = [np.load(os.path.join(args.load_ref, "output_%d.npy" % i))
                        for i in range(n_out)]
    else:
        inputs = make_inputs(sigs, args)
    if args.print_input:
        for i, a in enumerate(inputs):
            print("The %s input %s:[%s] is: \n %s \n" % (ordinal(i + 1), sigs[i][2],
                                                        "x".join(map(str, a.shape)), a))
    feed = inputs
    if args.device_resident:
        feed = [omcuda.Tensor.from_numpy(a).to_device() for a in inputs]
        omcuda.synchronize()

    def run():
        outs = sess.run(feed)
        if args.device_resident:
            omcuda.synchronize()
        return outs

    print("Running inference ...")
    for i in range(args.warmup):
        t0 = time.perf_counter()
        outs = run()
        print("  {} warmup: {} seconds".format(ordinal(i + 1), time.perf_counter() - t0))
    perf = []
    for i in range(args.n_iteration):
        t0 = time.perf_counter()
        outs = run()
        perf.append(time.perf_counter() - t0)
        print("  {} iteration, {}, seconds".format(ordinal(i + 1), perf[-1]))
    if args.n_iteration > 1:
        for label, data in (("Statistics 1 (excluding warmup),", perf),
                            ("Statistics 2 (no warmup/quart.),",
                             data_without_top_bottom_quartile(perf, 25))):
            print("  {} min, {:.6e}, max, {:.6e}, mean, {:.6e}, stdev, {:.6e}".format(
                label, np.min(data), np.max(data), np.mean(data),
                np.std(data, dtype=np.float64)))
    outs = [o.numpy() if isinstance(o, omcuda.Tensor) else o for o in outs]
    if args.print_output:
        for i, o in enumerate(outs):
            print("The %s output [%s] is: \n %s \n" % (ordinal(i + 1),
                                                      "x".join(map(str, o.shape)), o))
    if args.save_ref:
        os.makedirs(args.save_ref, exist_ok=True)
        for i, a in enumerate(inputs):
            np.save(os.path.join(args.save_ref, "input_%d.npy" % i), a)
        for i, o in enumerate(outs):
            np.save(os.path.join(args.save_ref, "output_%d.npy" % i), o)
        print("Saved inputs and outputs into", args.save_ref)
    if args.verify:
        rtol, atol = float(args.rtol), float(args.atol)
        total = 0
        for i, (o, r) in enumerate(zip(outs, ref_outs)):
            print("Verifying value of {}:{}".format("output_%d" % i, list(o.shape)),
                  "using atol={}, rtol={} ...".format(atol, rtol))
            if o.shape != r.shape:
                sys.exit("  shape mismatch: %s vs %s" % (o.shape, r.shape))
            bad = ~np.isclose(o.astype(np.float64), r.astype(np.float64), rtol=rtol, atol=atol)
            n = int(bad.sum())
            total += n
            if n:
                idx = np.argwhere(bad)[0]
                print("  at {} mismatch {} (actual) vs {} (reference)".format(
                    tuple(idx), o[tuple(idx)], r[tuple(idx)]))
                print("  mismatched elements: {}/{}".format(n, o.size))
            else:
                print("  correct.\n")
        if total:
            sys.exit(1)
    sess.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
