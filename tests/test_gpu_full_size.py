"""Parity at the benchmark configurations' real geometry.  The checker is the
compiled reference CPU path (oracle/_ref, OpenBLAS build) on a few samples of
each network -- inference has no cross-sample coupling, so a slice of the batch
is an exact sub-problem -- plus size-independent properties on the full batch."""
import numpy as np
import pytest

from nebula_b200 import workloads
from tests.util import NET_TOL, logit_err

pytestmark = pytest.mark.gpu


def _reference_logits(wl, w, x):
    from oracle import oracle as O
    # the last [connected] layer: followed by [softmax] in the image networks, last in the LSTM cfg
    logits_layer = -2 if "[softmax]" in wl.cfg else -1
    if O.ref_binary("oblas") is not None:
        out, _ = O.run_reference(wl.cfg, w, x, recurrent=wl.recurrent, flavour="oblas", out_layer=logits_layer)
        return out
    if O.ref_binary("custom") is not None:
        out, _ = O.run_reference(wl.cfg, w, x, recurrent=wl.recurrent, flavour="custom", out_layer=logits_layer)
        return out
    return O.forward_network(wl.cfg, w, x, keep_all=True)[logits_layer].ravel()


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


CASES = [("alexnet", 16, 1), ("vgg16", 4, 3), ("resnet50", 4, 4)]


@pytest.mark.parametrize("name,batch,seed", CASES, ids=[c[0] for c in CASES])
def test_full_geometry_against_reference(handle, name, batch, seed):
    wl = workloads.WORKLOADS[name](batch=batch)
    if name == "resnet50":
        wl = workloads.resnet50(batch=batch)
    w = wl.make_weights(1000 * seed)
    x = wl.make_input(1000 * seed + 1)
    ref = _reference_logits(wl, w, x)
    for mode in ("tf32", "tf32x3"):
        got = _gpu_logits(handle, wl, w, x, mode)
        err = logit_err(got, ref, batch)
        print(f"{name} b{batch} {mode}: logits err {err:.3e}")
        assert np.isfinite(got).all()
        assert err <= NET_TOL[mode], f"{name} {mode}: {err:.3e}"
        assert (got.reshape(batch, -1).argmax(1) == ref.reshape(batch, -1).argmax(1)).all(), f"{name} {mode}: argmax"


def test_lstm_benchmark_geometry_against_reference(handle):
    """Two LSTM layers (1024 -> 1024) and the 10000-way projection; 32 steps of batch 16."""
    wl = workloads.lstm2(batch=16, time_steps=32)
    w = wl.make_weights(5000)
    x = wl.make_input(5001)
    ref = _reference_logits(wl, w, x)
    for mode in ("tf32", "tf32x3"):
        got = _gpu_logits(handle, wl, w, x, mode)
        err = logit_err(got, ref, 32 * 16)
        print(f"lstm2 T32 B16 {mode}: logits err {err:.3e}")
        assert err <= NET_TOL[mode]
        # 512 rows x 10000 near-uniform classes: a handful of top-1 ties sit inside the rounding noise
        assert (got.reshape(512, -1).argmax(1) == ref.reshape(512, -1).argmax(1)).mean() > 0.99


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
    probs = net.output().reshape(256, -1)
    net.close()
    assert np.isfinite(big).all(), "non-finite logits in the b256 run"
    assert np.allclose(probs.sum(1), 1.0, atol=1e-4), f"softmax rows sum to {probs.sum(1).min()}..{probs.sum(1).max()}"
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
