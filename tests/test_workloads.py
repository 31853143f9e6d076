"""Host-side logic: workload builders emit cfg text, weight streams and inputs in
the reference's formats, with the shapes and FLOP counts of the benchmark
configurations."""
import numpy as np
import pytest

from nebula_b200 import workloads
from oracle import oracle as O


@pytest.mark.parametrize("name", ["alexnet", "vgg16", "resnet50", "lstm2", "conv_a", "conv_b", "conv_c"])
def test_weight_stream_length_matches_the_cfg(name):
    wl = workloads.WORKLOADS[name](batch=2)
    net, layers = O.plan_network(wl.cfg)
    assert O.weight_count(layers) == wl.weight_count()
    assert int(np.prod(layers[-1].out_shape)) == wl.classes or layers[-1].kind == "softmax"


def test_vgg16_shapes_and_flops():
    wl = workloads.vgg16()
    net, layers = O.plan_network(wl.cfg)
    convs = [l for l in layers if l.kind == "convolutional"]
    assert len(convs) == 13 and [l.kind for l in layers].count("maxpool") == 5
    assert layers[17].out_shape == (512, 7, 7)
    assert [l.params["inp"] for l in layers if l.kind == "connected"] == [25088, 4096, 4096]
    assert wl.weight_count() == 138357544
    assert abs(wl.conv_flops_per_unit / 1e9 - 30.693) < 0.01
    assert abs(wl.flops_per_unit / 1e9 - 30.941) < 0.01


def test_alexnet_and_resnet_topology():
    a = workloads.alexnet()
    net, layers = O.plan_network(a.cfg)
    assert layers[0].out_shape == (96, 55, 55) and layers[7].out_shape == (256, 6, 6)
    assert abs(a.flops_per_unit / 1e9 - 2.271) < 0.01
    r = workloads.resnet50()
    net, layers = O.plan_network(r.cfg)
    assert sum(l.kind == "convolutional" for l in layers) == 49 and sum(l.kind == "shortcut" for l in layers) == 16
    assert layers[-3].out_shape == (2048, 1, 1)
    assert abs(r.flops_per_unit / 1e9 - 7.459) < 0.01


def test_lstm_workload():
    wl = workloads.lstm2()
    assert wl.recurrent and wl.input_shape == (128, 64, 1024) and wl.classes == 10000
    # gates 2*(in+H)*4H per step per layer, projection 2*H*classes per step
    assert abs(wl.flops_per_unit - 128 * (2 * 2 * 2048 * 4096 + 2 * 1024 * 10000)) < 1


def test_generators_are_deterministic_and_in_range():
    wl = workloads.vgg16(batch=1, height=32, width=32, fc=64, classes=10)
    assert np.array_equal(wl.make_weights(3), wl.make_weights(3))
    x = wl.make_input(4)
    assert x.dtype == np.float32 and x.min() >= 0.0 and x.max() < 1.0
    s = wl.with_batch(5)
    assert "batch=5" in s.cfg and s.input_shape[0] == 5 and s.weight_count() == wl.weight_count()
