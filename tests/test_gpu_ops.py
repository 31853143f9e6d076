"""Operator-level parity on the GPU: every C-ABI operator against the CPU oracle
on the same seeded inputs, in the three arithmetic modes."""
import zlib

import numpy as np
import pytest

from tests.util import assert_close, rel_err

pytestmark = pytest.mark.gpu

MODES = ["fp32", "tf32", "tf32x3"]


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def _bn(rng, n):
    return (rng.uniform(0.8, 1.2, n).astype(np.float32), (0.1 * rng.standard_normal(n)).astype(np.float32),
            rng.uniform(0.5, 1.5, n).astype(np.float32))


# (B, C, H, W, F, k, stride, pad, bn, act)
CONV_CASES = [
    (2, 3, 13, 11, 8, 3, 1, 1, False, "relu"),          # 3 input channels: CUDA-core path in every mode
    (3, 32, 9, 9, 16, 3, 1, 1, True, "leaky"),          # smallest tensor-core case, N tile tail
    (2, 64, 14, 14, 96, 3, 1, 1, False, "relu"),
    (4, 64, 8, 8, 64, 1, 1, 0, True, "linear"),         # 1x1
    (2, 48, 12, 10, 40, 5, 1, 2, False, "relu"),        # C not a multiple of 32 (zero-filled K tail)
    (2, 64, 15, 15, 32, 3, 2, 1, True, "relu"),         # stride 2 (TMA element strides)
    (1, 32, 23, 23, 24, 7, 2, 3, False, "leaky"),       # 7x7 stride 2
    (2, 32, 31, 31, 16, 11, 4, 0, False, "relu"),       # 11x11 stride 4
    (5, 128, 7, 7, 256, 3, 1, 1, False, "relu"),        # several images per pixel box
    (1, 32, 40, 36, 300, 3, 1, 0, False, "tanh"),       # no padding, F tail over 256
    (2, 64, 28, 42, 64, 3, 1, 1, False, "relu"),        # filter-column stages, ragged 16 x 8 boxes in both directions
    (1, 128, 33, 56, 160, 3, 1, 1, True, "leaky"),      # C=128, ragged tiles in H, filter tail
    (3, 32, 16, 28, 40, 3, 1, 0, False, "linear"),      # filter-column stages without padding
    (2, 64, 32, 48, 128, 3, 1, 1, True, "relu"),        # filter-column stages, two boxes per tile
    (2, 3, 24, 32, 24, 3, 1, 1, False, "relu"),         # row windows as one filter column per tile (one box)
    (2, 3, 32, 64, 64, 3, 1, 1, False, "relu"),         # row windows, two boxes per tile, two staging buffers per group
    (1, 4, 36, 48, 64, 3, 1, 1, True, "leaky"),         # four input channels, ragged in H
    (1, 3, 34, 34, 16, 3, 1, 0, False, "linear"),       # row windows without padding
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: "x".join(map(str, c)))
def test_conv2d_nchw(handle, mode, case):
    from nebula_b200 import api
    from oracle import oracle as O
    B, C, H, W, F, k, s, p, bn, act = case
    rng = np.random.default_rng(zlib.crc32(repr(case).encode()))
    x = rng.standard_normal((B, C, H, W), dtype=np.float32)
    w = (rng.standard_normal((F, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    bias = (0.1 * rng.standard_normal(F)).astype(np.float32)
    bnp = _bn(rng, F) if bn else None
    ref = O.conv_forward(x, w, bias, k, s, p, act, bnp)
    handle.set_math(mode)
    plan = api.Conv2d(handle, B, C, H, W, F, k, s, p, bn, act, api.LAYOUT_NCHW)
    plan.set_weights(w, bias, bnp)
    y = plan.forward(_t(x)).cpu().numpy()
    handle.synchronize()
    plan.close()
    assert y.shape == ref.shape
    # a saturating activation turns the pre-activation error into error relative to 1
    assert_close(y, ref, mode, f"conv {case}", factor=3.0 if act == "tanh" else 1.0)


@pytest.mark.parametrize("mode", MODES)
def test_conv2d_nhwc_layout(handle, mode):
    from nebula_b200 import api
    from oracle import oracle as O
    rng = np.random.default_rng(5)
    B, C, H, W, F = 2, 64, 10, 12, 48
    x = rng.standard_normal((B, C, H, W), dtype=np.float32)
    w = (rng.standard_normal((F, C, 3, 3)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(F).astype(np.float32)
    ref = O.conv_forward(x, w, bias, 3, 1, 1, "relu")
    handle.set_math(mode)
    plan = api.Conv2d(handle, B, C, H, W, F, 3, 1, 1, False, "relu", api.LAYOUT_NHWC)
    plan.set_weights(_t(w), _t(bias))          # device-resident weights
    y = plan.forward(_t(x.transpose(0, 2, 3, 1))).cpu().numpy().transpose(0, 3, 1, 2)
    handle.synchronize()
    plan.close()
    assert_close(y, ref, mode, "conv nhwc")


FC_CASES = [(1, 32, 8, False, "linear"), (16, 256, 100, False, "relu"), (128, 512, 256, True, "leaky"),
            (33, 200, 77, False, "logistic"), (7, 50, 19, True, "tanh"), (256, 1024, 1000, False, "linear"),
            (200, 96, 513, False, "relu"),
            (32, 4096, 1000, False, "relu"), (64, 8192, 512, True, "leaky")]      # long K, few rows: split-K path


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", FC_CASES, ids=lambda c: "x".join(map(str, c)))
def test_connected(handle, mode, case):
    from nebula_b200 import api
    from oracle import oracle as O
    B, inp, out, bn, act = case
    rng = np.random.default_rng(inp * 7 + out)
    x = rng.standard_normal((B, inp), dtype=np.float32)
    w = (rng.standard_normal((out, inp)) / np.sqrt(inp)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(out)).astype(np.float32)
    bnp = _bn(rng, out) if bn else None
    ref = O.connected_forward(x, w, bias, act, bnp)
    handle.set_math(mode)
    plan = api.Connected(handle, B, inp, out, bn, act)
    plan.set_weights(w, bias, bnp)
    y = plan.forward(_t(x)).cpu().numpy()
    handle.synchronize()
    plan.close()
    assert_close(y, ref, mode, f"connected {case}")


POOL_CASES = [(2, 8, 8, 8, 2, 2, 0, "max"), (2, 5, 13, 11, 3, 2, 0, "max"), (1, 4, 7, 7, 3, 2, 1, "max"),
              (2, 16, 7, 7, 7, 7, 0, "avg"), (3, 6, 9, 10, 2, 2, 0, "avg"), (2, 3, 6, 6, 3, 1, 1, "avg"),
              (1, 7, 5, 5, 2, 1, 0, "max")]


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("case", POOL_CASES, ids=lambda c: "x".join(map(str, c)))
def test_pool(handle, layout, case):
    from nebula_b200 import api
    from oracle import oracle as O
    B, C, H, W, k, s, p, mode = case
    rng = np.random.default_rng(k * 100 + s)
    x = rng.standard_normal((B, C, H, W), dtype=np.float32)
    ref = O.pool_forward(x, k, s, p, mode == "max")
    if layout == "nchw":
        y = handle.pool(_t(x), k, s, p, mode, api.LAYOUT_NCHW).cpu().numpy()
    else:
        y = handle.pool(_t(x.transpose(0, 2, 3, 1)), k, s, p, mode, api.LAYOUT_NHWC).cpu().numpy().transpose(0, 3, 1, 2)
    handle.synchronize()
    assert np.array_equal(y, ref), f"pool {case} {layout}: max diff {np.abs(y - ref).max()}"


SHORTCUT_CASES = [((2, 8, 6, 6), (2, 8, 6, 6)), ((2, 4, 8, 8), (2, 16, 8, 8)), ((2, 16, 8, 8), (2, 32, 4, 4)),
                  ((1, 8, 4, 4), (1, 4, 8, 8)), ((3, 64, 14, 14), (3, 256, 14, 14))]


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("shapes", SHORTCUT_CASES, ids=str)
def test_shortcut(handle, layout, shapes):
    from nebula_b200 import api
    from oracle import oracle as O
    conn_s, prev_s = shapes
    rng = np.random.default_rng(11)
    conn = rng.standard_normal(conn_s, dtype=np.float32)
    prev = rng.standard_normal(prev_s, dtype=np.float32)
    ref = O.shortcut_forward(prev, conn, "leaky")
    if layout == "nchw":
        y = handle.shortcut(_t(prev), _t(conn), "leaky", api.LAYOUT_NCHW).cpu().numpy()
    else:
        y = handle.shortcut(_t(prev.transpose(0, 2, 3, 1)), _t(conn.transpose(0, 2, 3, 1)), "leaky",
                            api.LAYOUT_NHWC).cpu().numpy().transpose(0, 3, 1, 2)
    handle.synchronize()
    assert np.array_equal(y, ref)


@pytest.mark.parametrize("act", ["elu", "hardtan", "leaky", "lhtan", "linear", "loggy", "logistic", "plse", "ramp",
                                 "relie", "relu", "stair", "tanh"])
def test_activations(handle, act):
    from oracle import oracle as O
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(1001).astype(np.float32) * 3,
                        np.array([0.0, -0.0, 1.0, -1.0, 4.0, -4.0, 5.5, -5.5, 80.0, -80.0, 1e-8], np.float32)])
    ref = O.activate(x, act)
    y = handle.activation(_t(x), act).cpu().numpy()
    handle.synchronize()
    # exp() of the two libms may differ in the last place of the double result
    assert np.allclose(y, ref, rtol=2e-7, atol=1e-38, equal_nan=True), f"{act}: {np.abs(y - ref).max()}"


def test_tanh_overflow_matches_cpu(handle):
    """The CPU formula (e^2x-1)/(e^2x+1) gives NaN once e^2x overflows a double."""
    from oracle import oracle as O
    x = np.array([300.0, 354.0, 356.0, 400.0, -400.0], np.float32)
    ref = O.activate(x, "tanh")
    y = handle.activation(_t(x), "tanh").cpu().numpy()
    assert np.array_equal(np.isnan(y), np.isnan(ref))
    assert np.allclose(y[~np.isnan(y)], ref[~np.isnan(ref)])


def test_bias_and_batchnorm_passes(handle):
    from oracle import oracle as O
    rng = np.random.default_rng(8)
    B, Cc, S = 3, 5, 7
    x = rng.standard_normal((B, Cc, S), dtype=np.float32)
    scale, mean, var = _bn(rng, Cc)
    bias = rng.standard_normal(Cc).astype(np.float32)
    t = _t(x)
    handle.batchnorm_normalize(t, _t(mean), _t(var), Cc, S, B)
    handle.batchnorm_scale_down(t, _t(scale), Cc, S, B)
    handle.forward_bias(t, _t(bias), Cc, S, B)
    handle.synchronize()
    # the same three passes through the oracle: a 1x1 convolution with identity weights
    w = np.eye(Cc, dtype=np.float32).reshape(Cc, Cc, 1, 1)
    ref = O.conv_forward(x.reshape(B, Cc, S, 1), w, bias, 1, 1, 0, "linear", (scale, mean, var)).reshape(B, Cc, S)
    assert np.allclose(t.cpu().numpy(), ref, rtol=3e-7, atol=1e-7)


@pytest.mark.parametrize("shape", [(4, 10), (3, 1000), (130, 37), (2, 10000)])
def test_softmax(handle, shape):
    from oracle import oracle as O
    rng = np.random.default_rng(shape[1])
    x = (rng.standard_normal(shape) * 4).astype(np.float32)
    ref = O.softmax_forward(x)
    y = handle.softmax(_t(x)).cpu().numpy()
    handle.synchronize()
    assert np.allclose(y, ref, rtol=5e-5, atol=1e-12)      # the oracle sums sequentially in fp32
    assert np.allclose(y.sum(1), 1.0, atol=1e-5)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_operator(handle, ta, tb):
    rng = np.random.default_rng(ta * 2 + tb)
    M, N, K = 37, 29, 53
    A = rng.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    Bm = rng.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    Cm = rng.standard_normal((M, N)).astype(np.float32)
    from oracle import oracle as O
    # padded leading dimensions, as the operator's callers may pass them
    lda, ldb, ldc = A.shape[1] + 3, Bm.shape[1] + 5, N + 2
    Ap = np.zeros((A.shape[0], lda), np.float32); Ap[:, :A.shape[1]] = A
    Bp = np.zeros((Bm.shape[0], ldb), np.float32); Bp[:, :Bm.shape[1]] = Bm
    Cp = np.full((M, ldc), 7.0, np.float32); Cp[:, :N] = Cm
    ref = O.gemm(ta, tb, M, N, K, 0.5, Ap, lda, Bp, ldb, 1.0, Cp, ldc).reshape(M, ldc)       # the reference's gemm<T>
    out = handle.gemm(ta, tb, M, N, K, 0.5, _t(Ap), lda, _t(Bp), ldb, 1.0, _t(Cp), ldc).cpu().numpy()
    handle.synchronize()
    assert np.array_equal(out[:, N:], Cp[:, N:]), "columns beyond N must not be touched"
    assert rel_err(out[:, :N], ref[:, :N]) < 1e-5
    f64 = 0.5 * ((A.T if ta else A).astype(np.float64) @ (Bm.T if tb else Bm).astype(np.float64)) + 1.0 * Cm
    assert rel_err(out[:, :N], f64) < 1e-5


def test_layout_roundtrip(handle):
    from nebula_b200 import api
    rng = np.random.default_rng(2)
    x = rng.standard_normal((3, 37, 5, 9), dtype=np.float32)
    nhwc = handle.layout_convert(_t(x), 3, 37, 5, 9, api.LAYOUT_NCHW)
    assert np.array_equal(nhwc.cpu().numpy(), x.transpose(0, 2, 3, 1))
    back = handle.layout_convert(nhwc, 3, 37, 5, 9, api.LAYOUT_NHWC)
    assert np.array_equal(back.cpu().numpy(), x)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", [(5, 3, 12, 8, False), (6, 4, 64, 32, False), (4, 2, 40, 36, True)], ids=str)
def test_lstm(handle, mode, case):
    from nebula_b200 import api
    from nebula_b200.workloads import NetBuilder
    from oracle import oracle as O
    T, B, inp, H, bn = case
    b = NetBuilder("l", B, input_size=inp, time_steps=T, bias_init="bias_n01")
    b.lstm(H, bn=bn, bound=0.3)
    wl = b.build("normal")
    w = wl.make_weights(21)
    x = wl.make_input(22)
    ref = O.forward_network(wl.cfg, w, x)[0]
    handle.set_math(mode)
    plan = api.Lstm(handle, T, B, inp, H, bn, "linear")
    plan.set_weights(w)
    out, cell = plan.forward(_t(x), want_cell=True)
    handle.synchronize()
    plan.close()
    assert_close(out.cpu().numpy(), ref, mode, f"lstm {case}")


@pytest.mark.parametrize("case", [(6, 16, 64, 64, False), (9, 64, 96, 256, True), (5, 128, 64, 1024, False),
                                  (2, 8, 32, 96, False), (7, 5, 40, 32, False), (4, 100, 64, 160, True)],
                         ids=lambda c: "x".join(map(str, c)))
def test_lstm_one_kernel_recurrence_is_bit_identical(handle, case, monkeypatch):
    """TF32 mode runs steps 1..T-1 as one cooperative kernel (weights resident in shared memory, a grid barrier per
    step); NEBULA_B200_LSTM_PERSISTENT=0 selects the launch-per-step path.  Same K order, same cell arithmetic:
    hidden and cell states must agree bit for bit."""
    import torch
    from nebula_b200 import api
    from nebula_b200.workloads import NetBuilder
    T, B, inp, H, bn = case
    b = NetBuilder("l", B, input_size=inp, time_steps=T, bias_init="bias_n01")
    b.lstm(H, bn=bn, bound=0.3)
    wl = b.build("normal")
    w = wl.make_weights(31)
    x = _t(wl.make_input(32))
    handle.set_math("tf32")
    plan = api.Lstm(handle, T, B, inp, H, bn, "linear")
    plan.set_weights(w)
    monkeypatch.setenv("NEBULA_B200_LSTM_PERSISTENT", "0")
    out0, cell0 = plan.forward(x, want_cell=True)
    out0, cell0 = out0.clone(), cell0.clone()
    monkeypatch.delenv("NEBULA_B200_LSTM_PERSISTENT")
    out1, cell1 = plan.forward(x, want_cell=True)
    handle.synchronize()
    plan.close()
    assert torch.isfinite(out1).all()
    assert torch.equal(out0, out1) and torch.equal(cell0, cell1)


def test_error_reporting(handle):
    """Bad arguments come back as status codes with a message, never as exits."""
    from nebula_b200 import api
    with pytest.raises(api.NebulaError) as e:
        api.Conv2d(handle, 1, 3, 4, 4, 8, 7, 1, 0, False, "relu")      # filter larger than the input
    assert e.value.code == 1
    plan = api.Connected(handle, 2, 8, 4, False, "relu")
    import torch
    with pytest.raises(api.NebulaError) as e:
        plan.forward(torch.zeros(2, 8, device="cuda"))                  # forward before set_weights
    assert e.value.code == 7
    plan.close()
    with pytest.raises(api.NebulaError) as e:
        api.Network(handle, "[net]\nbatch=1\nheight=4\nwidth=4\nchannels=1\n[bogus]\nx=1\n")
    assert e.value.code == 5


ROWWIN_CASES = [(2, 3, 20, 24, 32, 3, 1, 1, False, "relu"), (2, 3, 33, 31, 64, 7, 2, 3, True, "relu"),
                (1, 3, 51, 51, 24, 11, 4, 0, False, "relu"), (3, 1, 16, 18, 16, 5, 1, 2, False, "leaky"),
                (2, 4, 12, 12, 40, 3, 2, 1, False, "linear")]


@pytest.mark.parametrize("mode", ["tf32", "tf32x3"])
@pytest.mark.parametrize("case", ROWWIN_CASES, ids=lambda c: "x".join(map(str, c)))
@pytest.mark.parametrize("route", ["1", "0"])
def test_conv2d_row_window_and_gather_routes(handle, mode, case, route, monkeypatch):
    """Layers with at most 4 input channels through the row-window route (default) and through the in-kernel gather
    (NEBULA_B200_ROW_WINDOWS=0, read when the plan is created): same tolerance."""
    from nebula_b200 import api
    from oracle import oracle as O
    monkeypatch.setenv("NEBULA_B200_ROW_WINDOWS", route)
    B, C, H, W, F, k, s, p, bn, act = case
    rng = np.random.default_rng(zlib.crc32(repr(case).encode()) + 1)
    x = rng.standard_normal((B, C, H, W), dtype=np.float32)
    w = (rng.standard_normal((F, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    bias = (0.1 * rng.standard_normal(F)).astype(np.float32)
    bnp = _bn(rng, F) if bn else None
    ref = O.conv_forward(x, w, bias, k, s, p, act, bnp)
    handle.set_math(mode)
    plan = api.Conv2d(handle, B, C, H, W, F, k, s, p, bn, act, api.LAYOUT_NCHW)
    plan.set_weights(w, bias, bnp)
    y = plan.forward(_t(x)).cpu().numpy()
    handle.synchronize()
    plan.close()
    assert_close(y, ref, mode, f"row-window conv {case}")
