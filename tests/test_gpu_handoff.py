"""The steps either side of the forward pass: decoded 8-bit images in (the reference's load_data conversion,
models/networks/convolutional.cc:263-423), probabilities out, pipelined; graph replay; the per-layer entry points'
scratch sizing, fused forms and operand checks."""
import numpy as np
import pytest

from tests.nets import NETS, tiny_vgg
from tests.util import TOL, rel_err

pytestmark = pytest.mark.gpu


def reference_pack(images_u8):
    """convolutional.cc:386-398: data[c][h][w] = u8[h][w][c] / 255.0 (double, stored as float), then planes 0 and 2
    swapped for three channels."""
    x = (images_u8.astype(np.float64) / 255.0).astype(np.float32)        # [B,H,W,C]
    x = np.ascontiguousarray(x.transpose(0, 3, 1, 2))
    if x.shape[1] == 3:
        x = np.ascontiguousarray(x[:, ::-1])
    return x


@pytest.mark.parametrize("mode", ["tf32", "tf32x3", "fp32"])
@pytest.mark.parametrize("name", ["tiny_vgg", "toy"])
def test_u8_images_equal_the_packed_float_batch(handle, name, mode):
    """Device-side packing is bit-exact: the pass from 8-bit images gives the very logits of the pass from the
    reference's own float conversion of the same images."""
    import torch
    from nebula_b200 import api
    handle.set_math(mode)
    wl = NETS[name]()
    B, C, H, W = wl.input_shape
    rng = np.random.default_rng(11)
    img = rng.integers(0, 256, size=(B, H, W, C), dtype=np.uint8)
    net = api.Network(handle, wl.cfg)
    net.load_weights(wl.make_weights(12))
    net.forward(torch.from_numpy(reference_pack(img)).cuda())
    handle.synchronize()
    want = net.logits()
    net.forward_u8(torch.from_numpy(img).cuda())
    handle.synchronize()
    assert np.array_equal(net.logits(), want)
    net.close()


def test_pipelined_submissions_match_synchronous_passes(handle):
    """Three batches submitted back to back (copy of batch i+1 overlapping pass i, two slots) return what three
    synchronous passes return; 8-bit and float submissions agree."""
    import torch
    from nebula_b200 import api
    handle.set_math("tf32")
    wl = tiny_vgg(batch=4)
    B, C, H, W = wl.input_shape
    net = api.Network(handle, wl.cfg)
    net.load_weights(wl.make_weights(21))
    rng = np.random.default_rng(22)
    imgs = [rng.integers(0, 256, size=(B, H, W, C), dtype=np.uint8) for _ in range(3)]
    want = []
    for im in imgs:
        net.forward(torch.from_numpy(reference_pack(im)).cuda())
        handle.synchronize()
        want.append(net.output())
    pin_u8 = [torch.from_numpy(im).pin_memory() for im in imgs]
    pin_f = [torch.from_numpy(reference_pack(im)).pin_memory() for im in imgs]
    for pins, submit in ((pin_u8, net.submit_u8), (pin_f, net.submit_host)):
        outs = [torch.zeros(net.output_size, dtype=torch.float32).pin_memory() for _ in imgs]
        for p, o in zip(pins, outs):
            submit(p, o)
        net.wait()
        for o, w in zip(outs, want):
            assert np.array_equal(o.numpy(), w)
    net.close()


@pytest.mark.parametrize("name", ["tiny_vgg", "tiny_resnet", "tiny_lstm", "tiny_rnn"])
def test_graph_replay_is_bit_identical(handle, name):
    import torch
    from nebula_b200 import api
    handle.set_math("tf32")
    wl = NETS[name]()
    net = api.Network(handle, wl.cfg)
    net.load_weights(wl.make_weights(31))
    x = torch.from_numpy(wl.make_input(32)).cuda()
    net.forward(x)
    handle.synchronize()
    want = net.logits()
    n0 = handle.launch_count()
    net.forward(x)
    per_pass = handle.launch_count() - n0
    net.set_graph(True)
    for _ in range(4):      # first: eager (input seen), second: capture + replay, then replays
        net.forward(x)
    handle.synchronize()
    assert np.array_equal(net.logits(), want)
    assert handle.launch_count() - n0 == 5 * per_pass, "replayed passes count their kernels too"
    net.close()


def test_prepare_sizes_the_scratch_and_forward_allocates_nothing(handle):
    import torch
    from nebula_b200 import api
    handle.set_math("tf32")
    conv = api.Conv2d(handle, 4, 64, 20, 20, 96, 3, 1, 1, False, "relu")        # NCHW: needs both layout scratches
    rng = np.random.default_rng(5)
    conv.set_weights(torch.from_numpy(rng.standard_normal((96, 64, 3, 3), dtype=np.float32)).cuda(),
                     torch.zeros(96, device="cuda"))
    assert conv.workspace_size() == 0
    need = conv.prepare()
    assert need >= 4 * (4 * 64 * 20 * 20 + 4 * 96 * 20 * 20)
    x = torch.from_numpy(rng.standard_normal((4, 64, 20, 20), dtype=np.float32)).cuda()
    y = conv.forward(x)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    y = conv.forward(x)
    handle.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free0 == free1 and conv.workspace_size() == need
    conv.close()


@pytest.mark.parametrize("mode", ["tf32", "tf32x3"])
def test_fused_conv_entry_points_match_the_separate_layers(handle, mode):
    """nb_conv2d_forward_fused: conv + shortcut and conv + 2x2/2 max-pool in one kernel, bit-identical to
    nb_conv2d_forward followed by nb_shortcut_forward / nb_pool_forward."""
    import torch
    from nebula_b200 import api
    handle.set_math(mode)
    rng = np.random.default_rng(6)
    B, C, H, W, F = 3, 64, 12, 12, 128
    x = torch.from_numpy(rng.standard_normal((B, H, W, C), dtype=np.float32)).cuda()
    w = torch.from_numpy((rng.standard_normal((F, C, 1, 1)) / 8).astype(np.float32)).cuda()
    b = torch.from_numpy((0.1 * rng.standard_normal(F)).astype(np.float32)).cuda()
    conn = torch.from_numpy(rng.standard_normal((B, 2 * H, 2 * W, 32), dtype=np.float32)).cuda()   # larger, fewer channels
    lin = api.Conv2d(handle, B, C, H, W, F, 1, 1, 0, False, "linear", layout=api.LAYOUT_NHWC)
    lin.set_weights(w, b)
    sep = handle.shortcut(lin.forward(x), conn, "leaky", layout=api.LAYOUT_NHWC)
    fused = lin.forward_fused(x, residual=conn, res_act="leaky")
    assert torch.equal(sep, fused)
    relu = api.Conv2d(handle, B, C, H, W, F, 1, 1, 0, False, "relu", layout=api.LAYOUT_NHWC)
    relu.set_weights(w, b)
    sep = handle.pool(relu.forward(x), 2, 2, 0, "max", layout=api.LAYOUT_NHWC)
    fused = relu.forward_fused(x, pool=True)
    assert torch.equal(sep, fused)
    lin.close()
    relu.close()
