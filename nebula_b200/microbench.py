"""Single-layer micro-benchmark through the C ABI (device-resident NHWC tensors).

    python -m nebula_b200.microbench conv --batch 64 --channels 256 --size 56 --filters 256 --k 3 --pad 1
    python -m nebula_b200.microbench fc --batch 256 --inputs 25088 --outputs 4096
    python -m nebula_b200.microbench lstm --batch 64 --inputs 1024 --outputs 1024 --steps 128
    python -m nebula_b200.microbench sweep        # the single-convolution sweep (batch 64, stride 1)
    python -m nebula_b200.microbench vgg_layers --batch 64    # a VGG-16 pass through the per-layer NCHW entries
    python -m nebula_b200.microbench passes --workload vgg16 --batch 256 --passes 2   # whole passes (for a profiler)

Prints one JSON line per case: device time per call (CUDA events on the stream
the kernels run on), algorithmic TFLOP/s and GB/s.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import api


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_conv(h, batch, channels, size, filters, k, stride, pad, math, iters=10, warmup=3, bn=False, act="relu"):
    h.set_math(math)
    plan = api.Conv2d(h, batch, channels, size, size, filters, k, stride, pad, bn, act, api.LAYOUT_NHWC)
    g = torch.Generator(device="cuda").manual_seed(1)
    w = torch.randn(filters, channels, k, k, device="cuda", generator=g) * (2.0 / (channels * k * k)) ** 0.5
    b = torch.zeros(filters, device="cuda")
    bnp = (torch.ones(filters, device="cuda"), torch.zeros(filters, device="cuda"), torch.ones(filters, device="cuda"))
    plan.set_weights(w, b, bnp if bn else None)
    x = torch.randn(batch, size, size, channels, device="cuda", generator=g)
    c, oh, ow = plan.output_dims()
    y = torch.empty(batch, oh, ow, c, device="cuda")
    fwd = lambda: h.check(h.lib.nb_conv2d_forward(plan.p, x.data_ptr(), y.data_ptr()))
    ms = _time(fwd, iters, warmup)
    h.synchronize()
    flops = 2.0 * batch * filters * oh * ow * channels * k * k
    nbytes = 4.0 * (x.numel() + y.numel() + w.numel())
    plan.close()
    return dict(op="conv", batch=batch, channels=channels, size=size, filters=filters, k=k, stride=stride, pad=pad,
                math=math, ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1), gbs=round(nbytes / ms / 1e6, 1))


def bench_fc(h, batch, inputs, outputs, math, iters=10, warmup=3):
    h.set_math(math)
    plan = api.Connected(h, batch, inputs, outputs, False, "relu")
    g = torch.Generator(device="cuda").manual_seed(2)
    plan.set_weights(torch.randn(outputs, inputs, device="cuda", generator=g) * (1.0 / inputs) ** 0.5,
                     torch.zeros(outputs, device="cuda"))
    x = torch.randn(batch, inputs, device="cuda", generator=g)
    y = torch.empty(batch, outputs, device="cuda")
    fwd = lambda: h.check(h.lib.nb_fc_forward(plan.p, x.data_ptr(), y.data_ptr()))
    ms = _time(fwd, iters, warmup)
    h.synchronize()
    flops = 2.0 * batch * inputs * outputs
    nbytes = 4.0 * (x.numel() + y.numel() + outputs * inputs)
    plan.close()
    return dict(op="fc", batch=batch, inputs=inputs, outputs=outputs, math=math, ms=round(ms, 4),
                tflops=round(flops / ms / 1e9, 1), gbs=round(nbytes / ms / 1e6, 1))


def bench_lstm(h, batch, inputs, hidden, steps, math, iters=10, warmup=3):
    """One LSTM layer over `steps` time steps: the input-side GEMM plus `steps - 1` recurrent GEMMs with the cell
    update in their epilogue."""
    import numpy as np
    from .workloads import NetBuilder
    h.set_math(math)
    b = NetBuilder("lstm", batch, input_size=inputs, time_steps=steps)
    b.lstm(hidden, bound=1.0 / 32)
    wl = b.build("normal")
    plan = api.Lstm(h, steps, batch, inputs, hidden, False, "linear")
    plan.set_weights(torch.from_numpy(np.ascontiguousarray(wl.make_weights(3))).cuda())
    x = torch.randn(steps * batch, inputs, device="cuda")
    out = torch.empty(steps, batch, hidden, device="cuda")
    fwd = lambda: h.check(h.lib.nb_lstm_forward(plan.p, x.data_ptr(), out.data_ptr(), None))
    ms = _time(fwd, iters, warmup)
    h.synchronize()
    flops = 2.0 * steps * batch * 4 * hidden * (inputs + hidden)
    plan.close()
    return dict(op="lstm", batch=batch, inputs=inputs, hidden=hidden, steps=steps, math=math, ms=round(ms, 4),
                us_per_step=round(ms * 1e3 / steps, 2), tflops=round(flops / ms / 1e9, 1))


def bench_vgg_per_layer(h, batch, math, iters=5, warmup=2):
    """One VGG-16 forward pass driven layer by layer through the per-layer entry points with the reference's own
    NCHW buffers (what a Nebula build bound as in INTEGRATION.md sections 2-4 executes), next to the network
    executor's pass over the same cfg."""
    import numpy as np
    from . import workloads
    h.set_math(math)
    wl = workloads.vgg16(batch=batch)
    w = wl.make_weights(1)
    x = torch.from_numpy(wl.make_input(2)).cuda()
    pos, c, hw = 0, 3, 224
    convs, fcs = [], []
    for width, reps in zip((64, 128, 256, 512, 512), (2, 2, 3, 3, 3)):
        for _ in range(reps):
            plan = api.Conv2d(h, batch, c, hw, hw, width, 3, 1, 1, False, "relu", api.LAYOUT_NCHW)
            nb, nw = width, width * c * 9
            plan.set_weights(np.ascontiguousarray(w[pos + nb:pos + nb + nw]), np.ascontiguousarray(w[pos:pos + nb]))
            plan.prepare()
            pos += nb + nw
            convs.append((plan, reps))
            c = width
        hw //= 2
    inp = 512 * 7 * 7
    for out, act in ((4096, "relu"), (4096, "relu"), (1000, "linear")):
        plan = api.Connected(h, batch, inp, out, False, act)
        plan.set_weights(np.ascontiguousarray(w[pos + out:pos + out + out * inp]), np.ascontiguousarray(w[pos:pos + out]))
        plan.prepare()
        pos += out + out * inp
        fcs.append(plan)
        inp = out

    def run():
        t, i = x, 0
        for reps in (2, 2, 3, 3, 3):
            for _ in range(reps):
                t = convs[i][0].forward(t)
                i += 1
            t = h.pool(t, 2, 2, 0, "max", api.LAYOUT_NCHW)
        t = t.reshape(batch, -1)
        for p in fcs:
            t = p.forward(t)
        return h.softmax(t)

    ms_layers = _time(run, iters, warmup)
    net = api.Network(h, wl.cfg)
    net.load_weights(w)
    ms_net = _time(lambda: net.forward(x), iters, warmup)
    h.synchronize()
    probs = run().cpu().numpy()
    # (not bit-identical: the executor feeds the first connected layer an NHWC tensor through permuted weight columns,
    # so its products are summed in another order)
    diff = float(np.abs(probs - net.output().reshape(batch, -1)).max())
    net.close()
    for p, _ in convs:
        p.close()
    for p in fcs:
        p.close()
    return dict(op="vgg16 layer by layer (NCHW entry points)", batch=batch, math=math, ms=round(ms_layers, 3),
                images_per_s=round(batch / ms_layers * 1e3, 1), executor_ms=round(ms_net, 3),
                executor_images_per_s=round(batch / ms_net * 1e3, 1), max_abs_diff_of_probabilities=diff)


def run_passes(h, workload, batch, math, passes):
    """`passes` forward passes of a benchmark network through the executor (the thing to put under a profiler)."""
    from . import workloads
    h.set_math(math)
    wl = workloads.WORKLOADS[workload](batch=batch)
    net = api.Network(h, wl.cfg)
    net.load_weights(wl.make_weights(1))
    x = torch.from_numpy(wl.make_input(2)).cuda()
    torch.cuda.synchronize()
    n0 = h.launch_count()
    ms = _time(lambda: net.forward(x), passes, 0)
    h.synchronize()
    out = dict(op="passes", workload=workload, batch=batch, math=math, passes=passes, ms_per_pass=round(ms, 4),
               launches_per_pass=(h.launch_count() - n0) // passes, launches_before=n0)
    net.close()
    return out


SWEEP = [(256, 56, 256, 3, 1), (512, 14, 512, 3, 1), (64, 56, 256, 1, 0)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["conv", "fc", "lstm", "sweep", "vgg", "vgg_layers", "passes"])
    ap.add_argument("--workload", default="vgg16")
    ap.add_argument("--passes", type=int, default=2)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--channels", type=int, default=256)
    ap.add_argument("--size", type=int, default=56)
    ap.add_argument("--filters", type=int, default=256)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=1)
    ap.add_argument("--inputs", type=int, default=4096)
    ap.add_argument("--outputs", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=128, help="lstm: time steps")
    ap.add_argument("--math", default="tf32")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    h = api.Handle(0, a.math)
    if a.op == "conv":
        print(json.dumps(bench_conv(h, a.batch, a.channels, a.size, a.filters, a.k, a.stride, a.pad, a.math, a.iters, a.warmup)))
    elif a.op == "fc":
        print(json.dumps(bench_fc(h, a.batch, a.inputs, a.outputs, a.math, a.iters, a.warmup)))
    elif a.op == "lstm":
        print(json.dumps(bench_lstm(h, a.batch, a.inputs, a.outputs, a.steps, a.math, a.iters, a.warmup)))
    elif a.op == "passes":
        print(json.dumps(run_passes(h, a.workload, a.batch, a.math, a.passes)))
    elif a.op == "vgg_layers":
        print(json.dumps(bench_vgg_per_layer(h, a.batch, a.math, a.iters, a.warmup)))
    elif a.op == "sweep":
        for c, s, f, k, p in SWEEP:
            print(json.dumps(bench_conv(h, a.batch, c, s, f, k, 1, p, a.math, a.iters, a.warmup)), flush=True)
    else:   # the distinct VGG-16 convolution shapes at the given batch
        for c, s, f in [(64, 224, 64), (64, 112, 128), (128, 112, 128), (128, 56, 256), (256, 56, 256), (256, 28, 512),
                        (512, 28, 512), (512, 14, 512)]:
            print(json.dumps(bench_conv(h, a.batch, c, s, f, 3, 1, 1, a.math, a.iters, a.warmup)), flush=True)
    h.close()


if __name__ == "__main__":
    main()
