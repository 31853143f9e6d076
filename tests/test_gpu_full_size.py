"""Parity at the benchmark configurations' real geometry and batch.  The checker is the
compiled reference CPU path (oracle/_ref, OpenBLAS build: the reference's default) -- at
the full batch on slices of it, since inference has no cross-sample coupling and the
reference needs about a second per image -- plus size-independent properties on the
full batch."""
import numpy as np
import pytest

from nebula_b200 import workloads
from tests.util import TOL, argmax_agrees, logit_err, net_tol, rel_err

pytestmark = pytest.mark.gpu


def _reference(wl, w, x, layer):
    from oracle import oracle as O
    for flavour in ("oblas", "custom"):
        if O.ref_binary(flavour) is not None:
            out, _ = O.run_reference(wl.cfg, w, x, recurrent=wl.recurrent, flavour=flavour, out_layer=layer)
            return out
    return O.forward_network(wl.cfg, w, x, keep_all=True)[layer].ravel()


def _reference_logits(wl, w, x):
    # the last [connected] layer: followed by [softmax] in the image networks, last in the recurrent cfgs
    return _reference(wl, w, x, -2 if "[softmax]" in wl.cfg else -1)


def _gpu_logits(handle, wl, w, x, mode):
    import torch
    from nebula_b200 import api
    handle.set_math(mode)
    net = api.Network(handle, wl.cfg)
    net.load_weights(w)
    net.forward(torch.from_numpy(x).cuda())
    handle.synchronize()
    out = net.logits()
    net.close()
    return out


def _check_logits(name, mode, got, ref, rows):
    err = logit_err(got, ref, rows)
    limit = net_tol(name, mode)
    ties, bad = argmax_agrees(got, ref, rows, limit)
    print(f"{name} rows={rows} {mode}: logits err {err:.3e} (limit {limit:.1e}); argmax ties within the bound: {ties}, differing: {len(bad)}")
    assert np.isfinite(got).all()
    assert err <= limit, f"{name} {mode}: {err:.3e} > {limit:.1e}"
    assert not bad, f"{name} {mode}: argmax differs beyond a tie in rows {bad[:10]}"
    return err


CASES = [("alexnet", 16, 1), ("vgg16", 4, 3), ("resnet50", 4, 4)]


@pytest.mark.parametrize("name,batch,seed", CASES, ids=[c[0] for c in CASES])
def test_full_geometry_against_reference(handle, name, batch, seed):
    wl = workloads.WORKLOADS[name](batch=batch)
    w = wl.make_weights(1000 * seed)
    x = wl.make_input(1000 * seed + 1)
    ref = _reference_logits(wl, w, x)
    for mode in ("tf32", "tf32x3"):
        _check_logits(name, mode, _gpu_logits(handle, wl, w, x, mode), ref, batch)


@pytest.mark.parametrize("case", ["a", "b", "c"])
def test_conv_sweep_at_batch_64_against_reference(handle, case):
    """The single-convolution sweep at its benchmark batch: (a) 256->256 3x3 @56x56, (b) 512->512 3x3 @14x14,
    (c) 64->256 1x1 @56x56, bias + ReLU fused; the checker is the reference's im2col + sgemm."""
    import torch
    from nebula_b200 import api
    wl = workloads.conv_micro(case, batch=64)
    w = wl.make_weights(2000 + ord(case))
    w[:wl.params[0].shape[0]] = 0.1 * np.random.default_rng(7).standard_normal(wl.params[0].shape[0])    # non-zero bias
    x = wl.make_input(2100 + ord(case))
    ref = _reference(wl, w, x, -1)
    for mode in ("tf32", "tf32x3"):
        handle.set_math(mode)
        net = api.Network(handle, wl.cfg)
        net.load_weights(w)
        net.forward(torch.from_numpy(x).cuda())
        handle.synchronize()
        got = net.layer_output(0, 64)
        net.close()
        err = rel_err(got, ref)
        print(f"conv_{case} b64 {mode}: rel err {err:.3e}")
        assert err <= TOL[mode], f"conv_{case} {mode}: {err:.3e}"


@pytest.mark.parametrize("name,seed", [("vgg16", 3000), ("resnet50", 4000)])
def test_batch_256_slices_against_reference(handle, name, seed):
    """The benchmark batch itself: rows of the 256-image pass against the compiled reference run on the first and the
    last eight images."""
    import torch
    from nebula_b200 import api
    full = workloads.WORKLOADS[name](batch=256)
    w = full.make_weights(seed)
    x = full.make_input(seed + 1)
    small = workloads.WORKLOADS[name](batch=8)
    refs = {lo: _reference_logits(small, w, x[lo:lo + 8].copy()) for lo in (0, 248)}
    for mode in ("tf32", "tf32x3"):
        handle.set_math(mode)
        net = api.Network(handle, full.cfg)
        net.load_weights(w)
        net.forward(torch.from_numpy(x).cuda())
        handle.synchronize()
        big = net.logits().reshape(256, -1)
        probs = net.output().reshape(256, -1)
        net.close()
        assert np.isfinite(big).all(), "non-finite logits in the b256 run"
        assert np.allclose(probs.sum(1), 1.0, atol=1e-4)
        for lo, ref in refs.items():
            _check_logits(name, mode, big[lo:lo + 8], ref, 8)


def test_lstm_benchmark_configuration_against_reference(handle):
    """Two LSTM layers (1024 -> 1024) and the 10000-way projection at the benchmark's T = 128, B = 64."""
    wl = workloads.lstm2(batch=64, time_steps=128)
    w = wl.make_weights(5000)
    x = wl.make_input(5001)
    ref = _reference_logits(wl, w, x)
    for mode in ("tf32", "tf32x3"):
        _check_logits("lstm2", mode, _gpu_logits(handle, wl, w, x, mode), ref, 128 * 64)


def test_vgg16_full_batch_equals_its_slices(handle):
    """Size-independent property at the benchmark batch: rows of the b256 run are bit-identical
    to the same images run as a batch of 8 (tile shapes change with the batch, the order of
    additions inside an output element does not)."""
    import torch
    from nebula_b200 import api
    handle.set_math("tf32")
    full = workloads.vgg16(batch=256)
    w = full.make_weights(3000)
    x = full.make_input(3001)
    net = api.Network(handle, full.cfg)
    net.load_weights(w)
    net.forward(torch.from_numpy(x).cuda())
    handle.synchronize()
    big = net.logits().reshape(256, -1)
    net.close()
    small = api.Network(handle, full.cfg, batch=8)
    small.load_weights(w)
    for lo in (0, 248):
        small.forward(torch.from_numpy(x[lo:lo + 8].copy()).cuda())
        handle.synchronize()
        got = small.logits().reshape(8, -1)
        diff = got != big[lo:lo + 8]
        assert not diff.any(), (f"images {lo}..{lo + 7}: {int(diff.sum())} logits differ in rows "
                                f"{np.nonzero(diff.any(1))[0].tolist()}, max |d| {np.abs(got - big[lo:lo + 8]).max():.3e}")
    small.close()
