"""Pins the CPU restatement (oracle/nebula_oracle.c) to the reference:
 * against the golden vectors under tests/golden/ (outputs of the compiled
   reference, committed with the script that made them), always;
 * against the compiled reference itself when oracle/_ref has been built.
The restatement keeps the loop order of the reference's in-tree GEMM, so it must
agree with the reference's `custom` build to the last bit, and with its OpenBLAS
build to fp32 summation noise."""
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import rel_err

GOLDEN = sorted(Path(__file__).resolve().parent.joinpath("golden").glob("*.npz"))


def _layers(z, flavour):
    keys = sorted(k for k in z.files if k.startswith(flavour + "_layer_"))
    return [z[k] for k in keys]


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_oracle_matches_golden_bitwise(path):
    z = np.load(path)
    outs = O.forward_network(str(z["cfg"]), z["weights"], z["input"], keep_all=True)
    ref = _layers(z, "custom")
    assert len(outs) == len(ref) > 0
    for i, (a, r) in enumerate(zip(outs, ref)):
        a = a.ravel()
        assert a.shape == r.shape, f"layer {i}"
        assert np.array_equal(a, r, equal_nan=True), f"{path.stem} layer {i}: max diff {np.nanmax(np.abs(a - r))}"


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_oracle_matches_openblas_reference(path):
    z = np.load(path)
    outs = O.forward_network(str(z["cfg"]), z["weights"], z["input"], keep_all=True)
    for i, (a, r) in enumerate(zip(outs, _layers(z, "oblas"))):
        finite = np.isfinite(r)
        assert rel_err(a.ravel()[finite], r[finite]) < 2e-6, f"{path.stem} layer {i}"


@pytest.mark.skipif(O.ref_binary("custom") is None, reason="oracle/_ref is not built on this machine")
def test_oracle_matches_live_reference():
    from tests.nets import tiny_resnet, tiny_vgg
    for make, seed in ((tiny_vgg, 5), (tiny_resnet, 6)):
        wl = make()
        w, x = wl.make_weights(seed), wl.make_input(seed + 1)
        outs = O.forward_network(wl.cfg, w, x, keep_all=True)
        ref, info = O.run_reference(wl.cfg, w, x, flavour="custom", dump_all=True, threads=4)
        assert info["layers"] == len(outs)
        for i, (a, r) in enumerate(zip(outs, ref)):
            assert np.array_equal(a.ravel(), r), f"{wl.name} layer {i}"


def test_cfg_parser_follows_reference_rules():
    secs = O.parse_cfg("# comment\n[ net ]\nBatch = 4\n batch=9\nHeight=8\n\n[Convolutional]\nActivation = ReLU\n")
    assert secs[0].name == "net" and secs[0].settings["batch"] == "4"      # first value of a repeated key wins
    assert secs[1].name == "Convolutional" and secs[1].settings["activation"] == "relu"


def test_pool_output_rule_and_defaults():
    """(H+2p)/stride with default padding (size-1)/2 (pooling_layer.cc:43-61)."""
    net, layers = O.plan_network("[net]\nbatch=1\nheight=13\nwidth=13\nchannels=2\n[maxpool]\nsize=3\nstride=2\n")
    assert layers[0].out_shape == (2, 7, 7)
    net, layers = O.plan_network("[net]\nbatch=1\nheight=55\nwidth=55\nchannels=2\n[maxpool]\nsize=3\nstride=2\npadding=0\n")
    assert layers[0].out_shape == (2, 27, 27)
    x = np.arange(2 * 25, dtype=np.float32).reshape(1, 2, 5, 5) - 30
    y = O.pool_forward(x, 2, 2, 1, True)       # windows hanging over the border see the -1e8 identity
    assert y.shape == (1, 2, 3, 3) and y[0, 0, 0, 0] == x[0, 0, 0, 0]
    ya = O.pool_forward(x, 3, 3, 1, False)     # divisor is size*size even where the window is clipped
    assert np.isclose(ya[0, 0, 0, 0], x[0, 0, :2, :2].sum() / 9.0)


def test_shortcut_channel_and_stride_mismatch():
    conn = np.ones((1, 2, 4, 4), np.float32)
    prev = np.zeros((1, 3, 2, 2), np.float32)
    y = O.shortcut_forward(prev, conn, "linear")
    assert y[0, :2].min() == 1 and y[0, 2].max() == 0      # only min(C) channels get the residual


def test_tanh_overflows_to_nan_like_the_reference():
    y = O.activate(np.array([400.0], np.float32), "tanh")
    assert np.isnan(y[0])
