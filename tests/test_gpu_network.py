"""Network-level parity on the GPU: cfg text + weight stream + input through the
network executor, compared layer by layer with the CPU oracle."""
import numpy as np
import pytest

from tests.nets import NETS, small_alexnet
from tests.util import NET_TOL, NET_TOL_EXCEPTIONS, assert_close, net_tol, rel_err

pytestmark = pytest.mark.gpu


def _run(handle, wl, mode, seed=1, fusion=False):
    import torch
    from nebula_b200 import api
    handle.set_math(mode)
    w = wl.make_weights(seed)
    x = wl.make_input(seed + 1)
    net = api.Network(handle, wl.cfg)
    assert net.weight_count == w.size
    net.set_fusion(fusion)          # unfused: every layer's output_data is materialised, as in the reference
    net.load_weights(w)
    net.forward(torch.from_numpy(x).cuda())
    handle.synchronize()
    return net, w, x


@pytest.mark.parametrize("name", list(NETS))
def test_network_fp32_every_layer(handle, name):
    """CUDA-core fp32 mode: every layer's output_data matches the oracle."""
    from oracle import oracle as O
    wl = NETS[name]()
    net, w, x = _run(handle, wl, "fp32")
    refs = O.forward_network(wl.cfg, w, x, keep_all=True)
    rows = x.shape[0] * (x.shape[1] if wl.recurrent else 1)
    assert net.num_layers == len(refs)
    for i, r in enumerate(refs):
        got = net.layer_output(i, rows)
        assert got.size == r.size, f"layer {i} ({net.layer_info(i)['type']}): size {got.size} vs {r.size}"
        assert_close(got, r, "fp32", f"{name} layer {i} ({net.layer_info(i)['type']})")
    net.close()


@pytest.mark.parametrize("mode", ["tf32", "tf32x3"])
@pytest.mark.parametrize("name", list(NETS))
def test_network_tensor_core_modes(handle, name, mode):
    from oracle import oracle as O
    wl = NETS[name]()
    net, w, x = _run(handle, wl, mode)
    refs = O.forward_network(wl.cfg, w, x, keep_all=True)
    rows = x.shape[0] * (x.shape[1] if wl.recurrent else 1)
    errs = [rel_err(net.layer_output(i, rows), r) for i, r in enumerate(refs)]
    logits = net.logits()
    li = max(i for i in range(net.num_layers) if net.layer_info(i)["type"] == "connected")
    e = assert_close(logits, refs[li], mode, f"{name} logits (per-layer errs {['%.1e' % v for v in errs]})", rows=rows,
                     tol={mode: net_tol(name, mode)})
    print(f"{name} {mode}: logits err {e:.2e}; per-layer {['%.1e' % v for v in errs]}")
    ref_l = refs[li].reshape(rows, -1)
    assert (logits.reshape(rows, -1).argmax(1) == ref_l.argmax(1)).all(), "argmax differs"
    net.close()


def test_alexnet_full_size_two_images(handle):
    """Full 3x227x227 AlexNet geometry (11x11 stride 4, 5x5, 3x3, 3/2 pools) on two images."""
    from oracle import oracle as O
    wl = small_alexnet(2)
    for mode in ("fp32", "tf32", "tf32x3"):
        net, w, x = _run(handle, wl, mode, seed=1001)
        ref = O.forward_network(wl.cfg, w, x, keep_all=True)
        logits = net.logits().reshape(2, -1)
        li = net.num_layers - 2
        e = assert_close(logits, ref[li], mode, f"alexnet logits {mode}", rows=2, tol=NET_TOL)
        print(f"alexnet {mode}: logits err {e:.2e}")
        assert (logits.argmax(1) == ref[li].reshape(2, -1).argmax(1)).all()
        probs = net.output().reshape(2, -1)
        assert np.allclose(probs.sum(1), 1.0, atol=1e-4)
        net.close()


@pytest.mark.parametrize("mode", ["tf32", "tf32x3"])
@pytest.mark.parametrize("name", ["tiny_vgg", "toy", "mid_vgg", "tiny_resnet"])
def test_fused_layers_are_bit_identical(handle, name, mode):
    """conv + 2x2/2 max-pool and conv + shortcut run as one kernel give exactly what the separate
    kernels give; only the fused convolutions' own outputs are no longer kept."""
    from nebula_b200 import api
    wl = NETS[name](batch=5)
    a, w, x = _run(handle, wl, mode, fusion=False)
    b, _, _ = _run(handle, wl, mode, fusion=True)
    assert np.array_equal(a.logits(), b.logits())
    fused = 0
    for i in range(a.num_layers):
        try:
            got = b.layer_output(i, 5)
        except api.NebulaError as e:
            assert e.code == 3 and a.layer_info(i)["type"] == "convolutional"
            fused += 1
            continue
        assert np.array_equal(a.layer_output(i, 5), got), f"layer {i} ({a.layer_info(i)['type']})"
    assert fused > 0
    a.close()
    b.close()


def test_forward_host_matches_device_path(handle):
    import torch
    from nebula_b200 import api
    wl = NETS["tiny_vgg"]()
    net, w, x = _run(handle, wl, "tf32")
    dev = net.output()
    xin = torch.from_numpy(x).pin_memory()
    out = torch.empty(net.output_size, dtype=torch.float32).pin_memory()
    net.forward_host(xin, out)
    assert np.array_equal(out.numpy(), dev)
    net.close()


def test_weight_stream_length_is_checked(handle):
    from nebula_b200 import api
    wl = NETS["toy"]()
    net = api.Network(handle, wl.cfg)
    w = wl.make_weights(1)
    with pytest.raises(api.NebulaError) as e:
        net.load_weights(w[:-1].copy())
    assert e.value.code == 4
    net.close()


def test_batch_override_and_linearity_in_batch(handle):
    """Inference has no cross-sample coupling: a batch equals its halves."""
    import torch
    from nebula_b200 import api
    handle.set_math("tf32")
    wl = NETS["tiny_vgg"](batch=4)
    w = wl.make_weights(5)
    x = wl.make_input(6)
    full = api.Network(handle, wl.cfg)
    full.load_weights(w)
    full.forward(torch.from_numpy(x).cuda())
    a = full.logits().reshape(4, -1)
    half = api.Network(handle, wl.cfg, batch=2)
    half.load_weights(w)
    outs = []
    for i in range(2):
        half.forward(torch.from_numpy(x[2 * i:2 * i + 2].copy()).cuda())
        outs.append(half.logits().reshape(2, -1))
    handle.synchronize()
    assert np.array_equal(a, np.concatenate(outs))
    full.close()
    half.close()
