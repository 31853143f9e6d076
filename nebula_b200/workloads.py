"""Synthetic workloads in the reference's own formats.

Builds, for each benchmark configuration, the three artefacts a Nebula run
consumes: the ``network.cfg`` text (sections and keys as read by the
reference's network classes, models/networks/convolutional.cc:52-122 and
recurrent.cc:116-176), a weight stream in weight-file order (network.cc:99-122;
conv/connected blobs are bias, weight, then scale/mean/variance when
batch-normalised; an LSTM holds eight connected blobs iW,fW,oW,cW,iU,fU,oU,cU,
lstm_layer.cc:194-206) and a seeded input batch (NCHW images, or time-major
[T,B,in] sequences as in recurrent.cc:197).

The reference evaluates on ImageNet / PTB with downloaded weights; neither is
available offline, so inputs and weights are seeded synthetic tensors with the
same shapes and value ranges (images uniform [0,1) like uint8/255, He-normal
weights).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    init: str            # "he", "zeros", "uniform", "bn_scale", "bn_mean", "bn_var", "bias_n01"
    fan_in: int = 1
    bound: float = 0.0


@dataclass
class Workload:
    name: str
    cfg: str
    params: list
    input_shape: tuple           # NCHW, or (T,B,in) for recurrent nets
    input_dist: str              # "uniform01" | "normal"
    recurrent: bool
    classes: int
    flops_per_unit: float        # algorithmic FLOPs per image (or per sequence)
    conv_flops_per_unit: float = 0.0
    unit: str = "images"
    layer_flops: list = field(default_factory=list)   # (kind, flops per unit) per weighted layer

    @property
    def batch(self):
        return self.input_shape[1] if self.recurrent else self.input_shape[0]

    def weight_count(self):
        return int(sum(int(np.prod(p.shape)) for p in self.params))

    def make_weights(self, seed: int) -> np.ndarray:
        """One flat little-endian fp32 stream in weight-file order.  Draw order
        is the file order, one generator per workload (PCG64)."""
        rng = np.random.default_rng(seed)
        out = np.empty(self.weight_count(), np.float32)
        pos = 0
        for p in self.params:
            n = int(np.prod(p.shape))
            if p.init == "he":
                a = rng.standard_normal(n, dtype=np.float32) * np.float32(np.sqrt(2.0 / p.fan_in))
            elif p.init == "zeros":
                a = np.zeros(n, np.float32)
            elif p.init == "uniform":
                a = rng.uniform(-p.bound, p.bound, n).astype(np.float32)
            elif p.init == "bn_scale":
                a = rng.uniform(0.8, 1.2, n).astype(np.float32)
            elif p.init == "bn_mean" or p.init == "bias_n01":
                a = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.1))
            elif p.init == "bn_var":
                a = rng.uniform(0.5, 1.5, n).astype(np.float32)
            else:
                raise ValueError(p.init)
            out[pos:pos + n] = a
            pos += n
        return out

    def make_input(self, seed: int, batch: int | None = None) -> np.ndarray:
        rng = np.random.default_rng(seed)
        shape = list(self.input_shape)
        if batch is not None:
            shape[1 if self.recurrent else 0] = batch
        if self.input_dist == "uniform01":
            return rng.random(tuple(shape), dtype=np.float32)
        return rng.standard_normal(tuple(shape), dtype=np.float32)

    def with_batch(self, batch: int) -> "Workload":
        """Same network with the [net] batch rewritten (per-GPU shard size)."""
        lines = []
        for ln in self.cfg.splitlines():
            lines.append(f"batch={batch}" if ln.replace(" ", "").startswith("batch=") else ln)
        shape = list(self.input_shape)
        shape[1 if self.recurrent else 0] = batch
        return Workload(self.name, "\n".join(lines) + "\n", self.params, tuple(shape), self.input_dist,
                        self.recurrent, self.classes, self.flops_per_unit, self.conv_flops_per_unit, self.unit,
                        self.layer_flops)


class NetBuilder:
    """Emits cfg sections while tracking shapes with the reference's rules."""

    def __init__(self, name, batch, channels=None, height=None, width=None, input_size=None, time_steps=None,
                 bias_init="zeros"):
        self.name = name
        self.recurrent = input_size is not None
        self.lines = ["[net]", f"batch={batch}"]
        if self.recurrent:
            self.lines += [f"input_size={input_size}", f"time_steps={time_steps}"]
            self.shape = (input_size,)
            self.input_shape = (time_steps, batch, input_size)
        else:
            self.lines += [f"height={height}", f"width={width}", f"channels={channels}"]
            self.shape = (channels, height, width)
            self.input_shape = (batch, channels, height, width)
        self.lines += ["num_threads=8", "num_iterations=1", ""]
        self.params: list[ParamSpec] = []
        self.shapes: list[tuple] = []
        self.flops = 0.0
        self.conv_flops = 0.0
        self.layer_flops = []
        self.bias_init = bias_init
        self.time_steps = time_steps or 1

    def _flat(self):
        return int(np.prod(self.shape))

    def _push(self, shape):
        self.shape = shape
        self.shapes.append(shape)

    def conv(self, filters, size, stride=1, padding=0, act="relu", bn=False):
        C, H, W = self.shape
        self.lines += ["[convolutional]"] + (["batch_normalize=1"] if bn else []) + [
            f"filters={filters}", f"size={size}", f"stride={stride}", f"padding={padding}", f"activation={act}", ""]
        i = len(self.shapes)
        fan = C * size * size
        self.params.append(ParamSpec(f"l{i}.bias", (filters,), self.bias_init))
        self.params.append(ParamSpec(f"l{i}.weight", (filters, C, size, size), "he", fan))
        if bn:
            self.params += [ParamSpec(f"l{i}.scale", (filters,), "bn_scale"),
                            ParamSpec(f"l{i}.mean", (filters,), "bn_mean"),
                            ParamSpec(f"l{i}.var", (filters,), "bn_var")]
        OH, OW = (H + 2 * padding - size) // stride + 1, (W + 2 * padding - size) // stride + 1
        f = 2.0 * filters * OH * OW * fan
        self.flops += f
        self.conv_flops += f
        self.layer_flops.append(("conv", f))
        self._push((filters, OH, OW))
        return self

    def connected(self, output, act="relu", bn=False, init="he", bound=0.0):
        inp = self._flat()
        self.lines += ["[connected]"] + (["batch_normalize=1"] if bn else []) + [
            f"output={output}", f"activation={act}", ""]
        i = len(self.shapes)
        self.params.append(ParamSpec(f"l{i}.bias", (output,), self.bias_init))
        self.params.append(ParamSpec(f"l{i}.weight", (output, inp), init, inp, bound))
        if bn:
            self.params += [ParamSpec(f"l{i}.scale", (output,), "bn_scale"),
                            ParamSpec(f"l{i}.mean", (output,), "bn_mean"),
                            ParamSpec(f"l{i}.var", (output,), "bn_var")]
        f = 2.0 * inp * output * self.time_steps
        self.flops += f
        self.layer_flops.append(("fc", f))
        self._push((output,))
        return self

    def pool(self, kind, size, stride, padding=None):
        C, H, W = self.shape
        p = (size - 1) // 2 if padding is None else padding
        self.lines += [f"[{kind}]", f"size={size}", f"stride={stride}"] + (
            [f"padding={padding}"] if padding is not None else []) + [""]
        self._push((C, (H + 2 * p) // stride, (W + 2 * p) // stride))
        return self

    def maxpool(self, size, stride, padding=None):
        return self.pool("maxpool", size, stride, padding)

    def avgpool(self, size, stride, padding=None):
        return self.pool("avgpool", size, stride, padding)

    def shortcut(self, hops, act="relu"):
        self.lines += ["[shortcut]", f"hops={hops}", f"activation={act}", ""]
        self._push(self.shape)
        return self

    def dropout(self, probability=0.5):
        self.lines += ["[dropout]", f"probability={probability}", ""]
        self._push(self.shape)
        return self

    def softmax(self):
        self.lines += ["[softmax]", "groups=1", ""]
        self._push(self.shape)
        return self

    def lstm(self, output, act="linear", bn=False, bound=1.0 / 32):
        inp = self._flat()
        self.lines += ["[lstm]"] + (["batch_normalize=1"] if bn else []) + [
            f"output={output}", f"activation={act}", ""]
        i = len(self.shapes)
        for g, gname in enumerate(("iW", "fW", "oW", "cW", "iU", "fU", "oU", "cU")):
            gin = output if g < 4 else inp
            self.params.append(ParamSpec(f"l{i}.{gname}.bias", (output,), self.bias_init))
            self.params.append(ParamSpec(f"l{i}.{gname}.weight", (output, gin), "uniform", gin, bound))
            if bn:
                self.params += [ParamSpec(f"l{i}.{gname}.scale", (output,), "bn_scale"),
                                ParamSpec(f"l{i}.{gname}.mean", (output,), "bn_mean"),
                                ParamSpec(f"l{i}.{gname}.var", (output,), "bn_var")]
        f = 2.0 * (inp + output) * 4 * output * self.time_steps
        self.flops += f
        self.layer_flops.append(("lstm", f))
        self._push((output,))
        return self

    def rnn(self, output, act="tanh", bn=False, bound=0.25):
        """Three connected blobs in file order input, hidden, output gate (rnn_layer.cc:69-73)."""
        inp = self._flat()
        self.lines += ["[rnn]"] + (["batch_normalize=1"] if bn else []) + [f"output={output}", f"activation={act}", ""]
        i = len(self.shapes)
        for gname, gin in (("in", inp), ("hid", output), ("out", output)):
            self.params.append(ParamSpec(f"l{i}.{gname}.bias", (output,), self.bias_init))
            self.params.append(ParamSpec(f"l{i}.{gname}.weight", (output, gin), "uniform", gin, bound))
            if bn:
                self.params += [ParamSpec(f"l{i}.{gname}.scale", (output,), "bn_scale"),
                                ParamSpec(f"l{i}.{gname}.mean", (output,), "bn_mean"),
                                ParamSpec(f"l{i}.{gname}.var", (output,), "bn_var")]
        f = 2.0 * (inp + 2 * output) * output * self.time_steps
        self.flops += f
        self.layer_flops.append(("rnn", f))
        self._push((output,))
        return self

    def rbm(self, output, act="logistic"):
        """Blob: hidden_bias, weight (rbm_layer.cc:150-157); forward is a connected layer (rbm_layer.cc:345-374)."""
        inp = self._flat()
        self.lines += ["[rbm]", f"output={output}", "k_step=1", f"activation={act}", ""]
        i = len(self.shapes)
        self.params.append(ParamSpec(f"l{i}.hidden_bias", (output,), self.bias_init))
        self.params.append(ParamSpec(f"l{i}.weight", (output, inp), "he", inp))
        f = 2.0 * inp * output
        self.flops += f
        self.layer_flops.append(("fc", f))
        self._push((output,))
        return self

    def build(self, input_dist="uniform01") -> Workload:
        return Workload(self.name, "\n".join(self.lines) + "\n", self.params, self.input_shape, input_dist,
                        self.recurrent, int(np.prod(self.shape)), self.flops, self.conv_flops,
                        "sequences" if self.recurrent else "images", self.layer_flops)


# ------------------------------------------------------------ named workloads
def alexnet(batch=16):
    """AlexNet as in benchmarks/alexnet_large/network.cfg (3x227x227, pools with
    explicit padding=0), ReLU, zero biases."""
    b = NetBuilder("alexnet", batch, 3, 227, 227)
    b.conv(96, 11, 4, 0).maxpool(3, 2, 0).conv(256, 5, 1, 2).maxpool(3, 2, 0)
    b.conv(384, 3, 1, 1).conv(384, 3, 1, 1).conv(256, 3, 1, 1).maxpool(3, 2, 0)
    b.connected(4096).dropout().connected(4096).dropout().connected(1000, act="linear").softmax()
    return b.build()


def vgg16(batch=256, height=224, width=224, fc=4096, classes=1000, widths=(64, 128, 256, 512, 512)):
    """VGG-16 as in benchmarks/vgg_large/network.cfg: 13 conv3x3 p1 ReLU, five
    2x2/2 max-pools, FC 25088-4096-4096-1000 with dropout (a no-op at inference)."""
    b = NetBuilder("vgg16", batch, 3, height, width)
    for w, reps in zip(widths, (2, 2, 3, 3, 3)):
        for _ in range(reps):
            b.conv(w, 3, 1, 1)
        b.maxpool(2, 2, 0)
    b.connected(fc).dropout().connected(fc).dropout().connected(classes, act="linear").softmax()
    return b.build()


def resnet50(batch=256, height=224, width=224, act="relu", base=64, blocks=(3, 4, 6, 3), classes=1000):
    """ResNet-50 in the reference's topology (benchmarks/resnet_large/network.cfg):
    conv7x7/2, maxpool 3/2 p0, bottlenecks {1x1 w, 3x3 w (stride 2 on the first
    block of stages 3-5), 1x1 4w linear, shortcut hops=4 + activation} with no
    projection convolutions (the residual covers min(C) channels), avgpool 7/7,
    FC.  Every conv is batch-normalised; beta is carried by the layer bias."""
    b = NetBuilder("resnet50", batch, 3, height, width, bias_init="bias_n01")
    b.conv(base, 7, 2, 3, act, bn=True).maxpool(3, 2, 0)
    for stage, reps in enumerate(blocks):
        w = base * (2 ** stage)
        for r in range(reps):
            stride = 2 if (stage > 0 and r == 0) else 1
            b.conv(w, 1, 1, 0, act, bn=True).conv(w, 3, stride, 1, act, bn=True)
            b.conv(4 * w, 1, 1, 0, "linear", bn=True).shortcut(4, act)
    b.avgpool(b.shape[1], b.shape[1], 0)
    b.connected(classes, act="linear").softmax()
    return b.build()


def lstm2(batch=64, time_steps=128, input_size=1024, hidden=1024, classes=10000, layers=2):
    """Two LSTM layers and a projection applied to every time step (a
    [connected] after [lstm] sees T*B rows, recurrent.cc:134-139)."""
    b = NetBuilder("lstm2", batch, input_size=input_size, time_steps=time_steps)
    for _ in range(layers):
        b.lstm(hidden)
    b.connected(classes, act="linear", init="uniform", bound=1.0 / 32)
    return b.build("normal")


def rnn2(batch=32, time_steps=16, input_size=256, hidden=256, classes=1000, layers=2, act="tanh", bn=False):
    """Vanilla RNN layers and a projection, the shape of benchmarks/rnn_*/network.cfg."""
    b = NetBuilder("rnn2", batch, input_size=input_size, time_steps=time_steps)
    for _ in range(layers):
        b.rnn(hidden, act, bn=bn, bound=1.0 / np.sqrt(hidden))
    b.connected(classes, act="linear", init="uniform", bound=1.0 / np.sqrt(hidden))
    return b.build("normal")


def dbn(batch=32, height=128, width=128, channels=3, hidden=(2000, 1000, 500, 30), classes=62):
    """Deep belief network at inference, the shape of benchmarks/dbn_large/network.cfg: [rbm] layers (logistic)
    and a linear [connected] classifier."""
    b = NetBuilder("dbn", batch, channels, height, width)
    for h in hidden:
        b.rbm(h, "logistic")
    b.connected(classes, act="linear").softmax()
    return b.build()


def conv_micro(case="a", batch=64):
    """Single-convolution sweep, stride 1, fused bias + ReLU."""
    cin, cout, k, p, hw = {"a": (256, 256, 3, 1, 56), "b": (512, 512, 3, 1, 14), "c": (64, 256, 1, 0, 56)}[case]
    b = NetBuilder(f"conv_{case}", batch, cin, hw, hw)
    b.conv(cout, k, 1, p)
    return b.build("normal")


WORKLOADS = {"alexnet": alexnet, "vgg16": vgg16, "resnet50": resnet50, "lstm2": lstm2, "rnn2": rnn2, "dbn": dbn,
             "conv_a": lambda batch=64: conv_micro("a", batch), "conv_b": lambda batch=64: conv_micro("b", batch),
             "conv_c": lambda batch=64: conv_micro("c", batch)}
