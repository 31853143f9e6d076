"""ctypes binding of ``libnebula_b200.so`` (the C ABI in ``include/nebula_b200.h``)
and thin Python mirrors of the reference's network / layer objects.

PyTorch is used only for device memory and streams: every compute call goes
through the C ABI into the hand-written sm_100a kernels.  There is no CPU or
eager fallback: if the library is missing or the device is not a B200 the calls
raise.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libnebula_b200.so"

MATH_TF32, MATH_TF32X3, MATH_FP32 = 0, 1, 2
MATH_MODES = {"tf32": MATH_TF32, "tf32x3": MATH_TF32X3, "fp32": MATH_FP32}
LAYOUT_NCHW, LAYOUT_NHWC = 0, 1
POOL_MAX, POOL_AVG = 0, 1
MEM_HOST, MEM_DEVICE = 0, 1
ACT = {"elu": 1, "hardtan": 2, "leaky": 3, "lhtan": 4, "linear": 5, "loggy": 6, "logistic": 7, "plse": 8,
       "ramp": 9, "relie": 10, "relu": 11, "stair": 12, "tanh": 13}
STATUS = {0: "NB_OK", 1: "NB_ERR_INVALID_ARG", 2: "NB_ERR_CUDA", 3: "NB_ERR_UNSUPPORTED", 4: "NB_ERR_WEIGHTS",
          5: "NB_ERR_CONFIG", 6: "NB_ERR_DEVICE_TIMEOUT", 7: "NB_ERR_NO_WEIGHTS"}
# the reference's layer_type_t codes (common/def.h:28-42)
LAYER_TYPES = {1: "connected", 2: "convolutional", 3: "cost", 4: "dropout", 5: "avgpool", 6: "maxpool",
               7: "shortcut", 8: "softmax", 9: "rnn", 10: "lstm", 11: "rbm"}


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "channels", "height", "width", "filters", "size", "stride",
                                       "padding", "batch_normalize", "activation", "layout")]


class FcDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "inputs", "outputs", "batch_normalize", "activation")]


class PoolDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "channels", "height", "width", "size", "stride", "padding",
                                       "mode", "layout")]


class ShortcutDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "conn_channels", "conn_height", "conn_width", "out_channels",
                                       "out_height", "out_width", "activation", "layout")]


class LstmDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("time_steps", "batch", "inputs", "hidden", "batch_normalize", "activation")]


class RnnDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("time_steps", "batch", "inputs", "hidden", "batch_normalize", "activation")]


class ConvFusion(C.Structure):
    _fields_ = [("residual", C.c_void_p), ("res_channels", C.c_int), ("res_height", C.c_int), ("res_width", C.c_int),
                ("res_activation", C.c_int), ("pool_out", C.c_void_p)]


class Profile(C.Structure):
    _fields_ = [("tc_ms", C.c_double), ("tc_flops", C.c_double), ("tc_launches", C.c_ulonglong),
                ("simt_ms", C.c_double), ("simt_flops", C.c_double), ("simt_launches", C.c_ulonglong),
                ("halo_ms", C.c_double), ("halo_flops", C.c_double), ("halo_launches", C.c_ulonglong)]


class LayerInfo(C.Structure):
    _fields_ = [("type", C.c_int), ("channels", C.c_int), ("height", C.c_int), ("width", C.c_int),
                ("size", C.c_size_t), ("activation", C.c_int)]


class NebulaError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"{STATUS.get(code, code)}: {message}")
        self.code = code


_FP = C.POINTER(C.c_float)
_VP = C.c_void_p

# name -> (restype, argtypes); every symbol include/nebula_b200.h declares
SIGNATURES = {
    "nb_create": (C.c_int, [C.c_int, C.POINTER(_VP)]),
    "nb_destroy": (C.c_int, [_VP]),
    "nb_last_error": (C.c_char_p, [_VP]),
    "nb_set_stream": (C.c_int, [_VP, _VP]),
    "nb_set_math_mode": (C.c_int, [_VP, C.c_int]),
    "nb_get_math_mode": (C.c_int, [_VP, C.POINTER(C.c_int)]),
    "nb_synchronize": (C.c_int, [_VP]),
    "nb_launch_count": (C.c_int, [_VP, C.POINTER(C.c_ulonglong)]),
    "nb_profile_begin": (C.c_int, [_VP]),
    "nb_profile_end": (C.c_int, [_VP, C.POINTER(Profile)]),
    "nb_conv2d_plan_create": (C.c_int, [_VP, C.POINTER(ConvDesc), C.POINTER(_VP)]),
    "nb_conv2d_set_weights": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, C.c_int]),
    "nb_conv2d_forward": (C.c_int, [_VP, _VP, _VP]),
    "nb_conv2d_forward_fused": (C.c_int, [_VP, _VP, _VP, C.POINTER(ConvFusion)]),
    "nb_plan_output_dims": (C.c_int, [_VP, C.POINTER(C.c_int * 3)]),
    "nb_plan_prepare": (C.c_int, [_VP]),
    "nb_workspace_size": (C.c_size_t, [_VP]),
    "nb_plan_destroy": (C.c_int, [_VP]),
    "nb_fc_plan_create": (C.c_int, [_VP, C.POINTER(FcDesc), C.POINTER(_VP)]),
    "nb_fc_set_weights": (C.c_int, [_VP, _VP, _VP, _VP, _VP, _VP, C.c_int]),
    "nb_fc_forward": (C.c_int, [_VP, _VP, _VP]),
    "nb_fc_forward_static": (C.c_int, [_VP, _VP, _VP, _VP, C.c_int, C.c_int, C.c_int, C.c_int, _VP]),
    "nb_pool_forward": (C.c_int, [_VP, C.POINTER(PoolDesc), _VP, _VP]),
    "nb_shortcut_forward": (C.c_int, [_VP, C.POINTER(ShortcutDesc), _VP, _VP, _VP]),
    "nb_lstm_plan_create": (C.c_int, [_VP, C.POINTER(LstmDesc), C.POINTER(_VP)]),
    "nb_lstm_set_weights": (C.c_int, [_VP, _VP, C.c_size_t, C.c_int]),
    "nb_lstm_forward": (C.c_int, [_VP, _VP, _VP, _VP]),
    "nb_rnn_plan_create": (C.c_int, [_VP, C.POINTER(RnnDesc), C.POINTER(_VP)]),
    "nb_rnn_set_weights": (C.c_int, [_VP, _VP, C.c_size_t, C.c_int]),
    "nb_rnn_forward": (C.c_int, [_VP, _VP, _VP]),
    "nb_activation_forward": (C.c_int, [_VP, C.c_int, _VP, C.c_size_t]),
    "nb_forward_bias": (C.c_int, [_VP, _VP, _VP, C.c_uint, C.c_uint, C.c_uint]),
    "nb_batchnorm_normalize": (C.c_int, [_VP, _VP, _VP, _VP, C.c_uint, C.c_uint, C.c_uint]),
    "nb_batchnorm_scale_down": (C.c_int, [_VP, _VP, _VP, C.c_uint, C.c_uint, C.c_uint]),
    "nb_softmax_forward": (C.c_int, [_VP, _VP, _VP, C.c_int, C.c_int]),
    "nb_gemm": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, _VP, C.c_int, _VP, C.c_int,
                          C.c_float, _VP, C.c_int]),
    "nb_layout_convert": (C.c_int, [_VP, _VP, _VP, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "nb_network_create": (C.c_int, [_VP, C.c_char_p, C.c_int, C.POINTER(_VP)]),
    "nb_network_load_weights": (C.c_int, [_VP, _VP, C.c_size_t, C.c_int]),
    "nb_network_load_weight_file": (C.c_int, [_VP, C.c_char_p]),
    "nb_network_weight_count": (C.c_size_t, [_VP]),
    "nb_network_forward": (C.c_int, [_VP, _VP]),
    "nb_network_forward_host": (C.c_int, [_VP, _VP, _VP]),
    "nb_network_submit_host": (C.c_int, [_VP, _VP, _VP]),
    "nb_network_submit_u8": (C.c_int, [_VP, _VP, _VP]),
    "nb_network_wait": (C.c_int, [_VP]),
    "nb_network_forward_u8": (C.c_int, [_VP, _VP]),
    "nb_network_set_graph": (C.c_int, [_VP, C.c_int]),
    "nb_network_workspace_size": (C.c_size_t, [_VP]),
    "nb_network_set_fusion": (C.c_int, [_VP, C.c_int]),
    "nb_network_num_layers": (C.c_int, [_VP]),
    "nb_network_layer_info": (C.c_int, [_VP, C.c_int, C.POINTER(LayerInfo)]),
    "nb_network_layer_output": (C.c_int, [_VP, C.c_int, _VP, C.c_int]),
    "nb_network_output": (C.c_int, [_VP, _VP, C.c_int]),
    "nb_network_logits": (C.c_int, [_VP, _VP, C.c_int]),
    "nb_network_output_size": (C.c_size_t, [_VP]),
    "nb_network_logits_size": (C.c_size_t, [_VP]),
    "nb_network_input_size": (C.c_size_t, [_VP]),
    "nb_network_destroy": (C.c_int, [_VP]),
}

_lib = None


def load_library(path: Path | None = None):
    """Loads the CUDA library; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path or LIB_PATH)
    if not p.exists():
        raise FileNotFoundError(f"{p} not found: build it with `python -m nebula_b200.build` "
                                "(there is no CPU fallback)")
    lib = C.CDLL(str(p))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the ABI is incomplete
        fn.restype, fn.argtypes = res, args
    if path is None:
        _lib = lib
    return lib


def _ptr(t, dtype="float32"):
    """Device (torch) or host (numpy) buffer -> raw address."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        assert t.dtype == np.dtype(dtype) and t.flags["C_CONTIGUOUS"]
        return t.ctypes.data
    assert t.dtype.__str__() == "torch." + dtype and t.is_contiguous(), f"expected a contiguous {dtype} tensor"
    return t.data_ptr()


def _mem(t):
    if isinstance(t, np.ndarray):
        return MEM_HOST
    return MEM_DEVICE if t.is_cuda else MEM_HOST


class Handle:
    """One per host thread and GPU (the reference's network_t holds the
    equivalent device state, models/networks/network.cc:44-51)."""

    def __init__(self, device: int = 0, math: str | int = "tf32"):
        self.lib = load_library()
        self.device = device
        h = _VP()
        rc = self.lib.nb_create(device, C.byref(h))
        if rc != 0:
            raise NebulaError(rc, (self.lib.nb_last_error(None) or b"").decode())
        self.h = h
        self.set_math(math)

    def check(self, rc):
        if rc != 0:
            raise NebulaError(rc, (self.lib.nb_last_error(self.h) or b"").decode())

    def set_math(self, math):
        self.check(self.lib.nb_set_math_mode(self.h, MATH_MODES[math] if isinstance(math, str) else int(math)))

    def set_stream(self, stream_ptr: int):
        self.check(self.lib.nb_set_stream(self.h, stream_ptr))

    def synchronize(self):
        self.check(self.lib.nb_synchronize(self.h))

    def launch_count(self) -> int:
        n = C.c_ulonglong()
        self.check(self.lib.nb_launch_count(self.h, C.byref(n)))
        return n.value

    def profile_begin(self):
        self.check(self.lib.nb_profile_begin(self.h))

    def profile_end(self) -> dict:
        p = Profile()
        self.check(self.lib.nb_profile_end(self.h, C.byref(p)))
        return {k: getattr(p, k) for k, _ in Profile._fields_}

    def close(self):
        if getattr(self, "h", None):
            self.lib.nb_destroy(self.h)
            self.h = None

    # ------------------------------------------------- stateless operators
    def pool(self, x, size, stride, padding, mode="max", layout=LAYOUT_NCHW):
        import torch
        if layout == LAYOUT_NCHW:
            B, Cc, H, W = x.shape
        else:
            B, H, W, Cc = x.shape
        OH, OW = (H + 2 * padding) // stride, (W + 2 * padding) // stride
        shape = (B, Cc, OH, OW) if layout == LAYOUT_NCHW else (B, OH, OW, Cc)
        y = torch.empty(shape, device=x.device, dtype=torch.float32)
        d = PoolDesc(B, Cc, H, W, size, stride, padding, POOL_MAX if mode == "max" else POOL_AVG, layout)
        self.check(self.lib.nb_pool_forward(self.h, C.byref(d), _ptr(x), _ptr(y)))
        return y

    def shortcut(self, prev, conn, act="linear", layout=LAYOUT_NCHW):
        import torch
        if layout == LAYOUT_NCHW:
            B, Co, Ho, Wo = prev.shape
            _, Ci, Hi, Wi = conn.shape
        else:
            B, Ho, Wo, Co = prev.shape
            _, Hi, Wi, Ci = conn.shape
        y = torch.empty_like(prev)
        d = ShortcutDesc(B, Ci, Hi, Wi, Co, Ho, Wo, ACT[act], layout)
        self.check(self.lib.nb_shortcut_forward(self.h, C.byref(d), _ptr(prev), _ptr(conn), _ptr(y)))
        return y

    def activation(self, x, act):
        """In place, like the reference's _<name>_activation_."""
        self.check(self.lib.nb_activation_forward(self.h, ACT[act], _ptr(x), x.numel()))
        return x

    def forward_bias(self, out, bias, channel, size, batch):
        self.check(self.lib.nb_forward_bias(self.h, _ptr(out), _ptr(bias), channel, size, batch))
        return out

    def batchnorm_normalize(self, out, mean, var, channel, size, batch):
        self.check(self.lib.nb_batchnorm_normalize(self.h, _ptr(out), _ptr(mean), _ptr(var), channel, size, batch))
        return out

    def batchnorm_scale_down(self, out, scale, channel, size, batch):
        self.check(self.lib.nb_batchnorm_scale_down(self.h, _ptr(out), _ptr(scale), channel, size, batch))
        return out

    def fc_forward_static(self, x, weight, bias, activation="linear", out=None):
        """Connected-layer forward through the entry point that allocates nothing
        (its scratch is a fixed array inside the library); device tensors only.
        Pass `out` to keep this wrapper from allocating the result tensor."""
        import torch
        batch, inputs = x.shape
        outputs = weight.shape[0]
        y = out if out is not None else torch.empty((batch, outputs), device=x.device, dtype=torch.float32)
        self.check(self.lib.nb_fc_forward_static(self.h, _ptr(x), _ptr(weight), _ptr(bias), batch, inputs, outputs,
                                                 ACT[activation], _ptr(y)))
        return y

    def softmax(self, x):
        import torch
        rows, classes = x.shape
        y = torch.empty_like(x)
        self.check(self.lib.nb_softmax_forward(self.h, _ptr(x), _ptr(y), rows, classes))
        return y

    def gemm(self, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, Cm, ldc):
        self.check(self.lib.nb_gemm(self.h, int(ta), int(tb), M, N, K, alpha, _ptr(A), lda, _ptr(B), ldb, beta,
                                    _ptr(Cm), ldc))
        return Cm

    def layout_convert(self, src, batch, channels, height, width, src_layout):
        import torch
        dst = torch.empty(src.numel(), device=src.device, dtype=torch.float32)
        self.check(self.lib.nb_layout_convert(self.h, _ptr(src), _ptr(dst), batch, channels, height, width, src_layout))
        return dst.view((batch, height, width, channels) if src_layout == LAYOUT_NCHW else
                        (batch, channels, height, width))


class _Plan:
    def __init__(self, handle: Handle):
        self.handle = handle
        self.p = _VP()

    def output_dims(self):
        d = (C.c_int * 3)()
        self.handle.check(self.handle.lib.nb_plan_output_dims(self.p, C.byref(d)))
        return tuple(d)

    def prepare(self):
        """Allocates the plan's scratch now (for the handle's math mode), so that forward calls allocate nothing."""
        self.handle.check(self.handle.lib.nb_plan_prepare(self.p))
        return self.workspace_size()

    def workspace_size(self) -> int:
        return self.handle.lib.nb_workspace_size(self.p)

    def close(self):
        if self.p:
            self.handle.lib.nb_plan_destroy(self.p)
            self.p = _VP()


class Conv2d(_Plan):
    """convolutional_layer_t: init -> plan, init_weight -> set_weights, _forward_ -> forward."""

    def __init__(self, handle, batch, channels, height, width, filters, size, stride=1, padding=0,
                 batch_normalize=False, activation="relu", layout=LAYOUT_NCHW):
        super().__init__(handle)
        self.desc = ConvDesc(batch, channels, height, width, filters, size, stride, padding, int(batch_normalize),
                             ACT[activation] if isinstance(activation, str) else activation, layout)
        handle.check(handle.lib.nb_conv2d_plan_create(handle.h, C.byref(self.desc), C.byref(self.p)))

    def set_weights(self, weight, bias, bn=None):
        s, m, v = bn if bn is not None else (None, None, None)
        self.handle.check(self.handle.lib.nb_conv2d_set_weights(self.p, _ptr(weight), _ptr(bias), _ptr(s), _ptr(m),
                                                                _ptr(v), _mem(weight)))

    def forward(self, x):
        import torch
        Cc, OH, OW = self.output_dims()
        B = self.desc.batch
        shape = (B, Cc, OH, OW) if self.desc.layout == LAYOUT_NCHW else (B, OH, OW, Cc)
        y = torch.empty(shape, device=x.device, dtype=torch.float32)
        self.handle.check(self.handle.lib.nb_conv2d_forward(self.p, _ptr(x), _ptr(y)))
        return y


    def forward_fused(self, x, residual=None, res_act="linear", pool=False):
        """NHWC plans: the following [shortcut] (residual: NHWC tensor of the connected layer) or 2x2/2 [maxpool]
        folded into this convolution's epilogue."""
        import torch
        Cc, OH, OW = self.output_dims()
        B = self.desc.batch
        f = ConvFusion()
        if residual is not None:
            _, rh, rw, rc = residual.shape
            f.residual, f.res_channels, f.res_height, f.res_width = _ptr(residual), rc, rh, rw
            f.res_activation = ACT[res_act]
        y = torch.empty((B, OH // 2, OW // 2, Cc) if pool else (B, OH, OW, Cc), device=x.device, dtype=torch.float32)
        if pool:
            f.pool_out = _ptr(y)
        self.handle.check(self.handle.lib.nb_conv2d_forward_fused(self.p, _ptr(x), None if pool else _ptr(y), C.byref(f)))
        return y


class Connected(_Plan):
    def __init__(self, handle, batch, inputs, outputs, batch_normalize=False, activation="relu"):
        super().__init__(handle)
        self.desc = FcDesc(batch, inputs, outputs, int(batch_normalize),
                           ACT[activation] if isinstance(activation, str) else activation)
        handle.check(handle.lib.nb_fc_plan_create(handle.h, C.byref(self.desc), C.byref(self.p)))

    def set_weights(self, weight, bias, bn=None):
        s, m, v = bn if bn is not None else (None, None, None)
        self.handle.check(self.handle.lib.nb_fc_set_weights(self.p, _ptr(weight), _ptr(bias), _ptr(s), _ptr(m),
                                                            _ptr(v), _mem(weight)))

    def forward(self, x):
        import torch
        y = torch.empty((self.desc.batch, self.desc.outputs), device=x.device, dtype=torch.float32)
        self.handle.check(self.handle.lib.nb_fc_forward(self.p, _ptr(x), _ptr(y)))
        return y


class Lstm(_Plan):
    def __init__(self, handle, time_steps, batch, inputs, hidden, batch_normalize=False, activation="linear"):
        super().__init__(handle)
        self.desc = LstmDesc(time_steps, batch, inputs, hidden, int(batch_normalize), ACT[activation])
        handle.check(handle.lib.nb_lstm_plan_create(handle.h, C.byref(self.desc), C.byref(self.p)))

    def set_weights(self, stream):
        self.handle.check(self.handle.lib.nb_lstm_set_weights(self.p, _ptr(stream), stream.size if isinstance(
            stream, np.ndarray) else stream.numel(), _mem(stream)))

    def forward(self, x, want_cell=False):
        import torch
        d = self.desc
        out = torch.empty((d.time_steps, d.batch, d.hidden), device=x.device, dtype=torch.float32)
        cell = torch.empty_like(out) if want_cell else None
        self.handle.check(self.handle.lib.nb_lstm_forward(self.p, _ptr(x), _ptr(out), _ptr(cell)))
        return (out, cell) if want_cell else out


class Rnn(_Plan):
    """rnn_layer_t: input, hidden and output gate as three connected layers of one section."""

    def __init__(self, handle, time_steps, batch, inputs, hidden, batch_normalize=False, activation="tanh"):
        super().__init__(handle)
        self.desc = RnnDesc(time_steps, batch, inputs, hidden, int(batch_normalize), ACT[activation])
        handle.check(handle.lib.nb_rnn_plan_create(handle.h, C.byref(self.desc), C.byref(self.p)))

    def set_weights(self, stream):
        self.handle.check(self.handle.lib.nb_rnn_set_weights(self.p, _ptr(stream), stream.size if isinstance(
            stream, np.ndarray) else stream.numel(), _mem(stream)))

    def forward(self, x):
        import torch
        d = self.desc
        out = torch.empty((d.time_steps, d.batch, d.hidden), device=x.device, dtype=torch.float32)
        self.handle.check(self.handle.lib.nb_rnn_forward(self.p, _ptr(x), _ptr(out)))
        return out


class Network:
    """Mirror of network_t: init from a network.cfg text, load a weight stream,
    forward over a batch (models/networks/network.cc:57-63,82-122)."""

    def __init__(self, handle: Handle, cfg_text: str, batch: int = 0):
        self.handle = handle
        self.n = _VP()
        handle.check(handle.lib.nb_network_create(handle.h, cfg_text.encode(), batch, C.byref(self.n)))
        lib = handle.lib
        self.num_layers = lib.nb_network_num_layers(self.n)
        self.weight_count = lib.nb_network_weight_count(self.n)
        self.input_size = lib.nb_network_input_size(self.n)
        self.output_size = lib.nb_network_output_size(self.n)
        self.logits_size = lib.nb_network_logits_size(self.n)

    def load_weights(self, stream):
        n = stream.size if isinstance(stream, np.ndarray) else stream.numel()
        self.handle.check(self.handle.lib.nb_network_load_weights(self.n, _ptr(stream), n, _mem(stream)))

    def load_weight_file(self, path):
        self.handle.check(self.handle.lib.nb_network_load_weight_file(self.n, str(path).encode()))

    def set_fusion(self, enable: bool):
        """Fusion on (default): conv + 2x2/2 max-pool run as one kernel and the conv's own output is not kept."""
        self.handle.check(self.handle.lib.nb_network_set_fusion(self.n, int(enable)))

    def layer_info(self, i):
        info = LayerInfo()
        self.handle.check(self.handle.lib.nb_network_layer_info(self.n, i, C.byref(info)))
        return dict(type=LAYER_TYPES.get(info.type, info.type), channels=info.channels, height=info.height,
                    width=info.width, size=info.size, activation=info.activation)

    def forward(self, x):
        """x: device tensor, NCHW [B,C,H,W] or time-major [T,B,in]."""
        assert x.numel() == self.input_size, f"input has {x.numel()} elements, network expects {self.input_size}"
        self.handle.check(self.handle.lib.nb_network_forward(self.n, _ptr(x)))

    def forward_host(self, x_host, out_host):
        """x_host/out_host: host buffers (numpy or pinned torch tensors); copies in, runs, copies out."""
        self.handle.check(self.handle.lib.nb_network_forward_host(self.n, _ptr(x_host), _ptr(out_host)))

    def submit_host(self, x_host, out_host):
        """Queues copy-in, forward and copy-out of one fp32 host batch and returns; at most two may be outstanding."""
        self.handle.check(self.handle.lib.nb_network_submit_host(self.n, _ptr(x_host), _ptr(out_host)))

    def submit_u8(self, images_host, out_host):
        """Same for decoded 8-bit images [B,H,W,C] (BGR for C = 3)."""
        assert images_host.numel() if hasattr(images_host, "numel") else images_host.size == self.input_size
        self.handle.check(self.handle.lib.nb_network_submit_u8(self.n, _ptr(images_host, "uint8"), _ptr(out_host)))

    def wait(self):
        self.handle.check(self.handle.lib.nb_network_wait(self.n))

    def forward_u8(self, images_dev):
        """One pass over decoded 8-bit images [B,H,W,C] that are on the device."""
        assert images_dev.numel() == self.input_size
        self.handle.check(self.handle.lib.nb_network_forward_u8(self.n, _ptr(images_dev, "uint8")))

    def set_graph(self, enable: bool):
        """Replay passes as CUDA graphs (from the second pass with the same input buffer on)."""
        self.handle.check(self.handle.lib.nb_network_set_graph(self.n, int(enable)))

    def workspace_size(self) -> int:
        return self.handle.lib.nb_network_workspace_size(self.n)

    def _fetch(self, fn, size, device):
        import torch
        if device is None:
            out = np.empty(size, np.float32)
            self.handle.check(fn(self.n, _ptr(out), MEM_HOST))
            return out
        out = torch.empty(size, device=device, dtype=torch.float32)
        self.handle.check(fn(self.n, _ptr(out), MEM_DEVICE))
        return out

    def output(self, device=None):
        return self._fetch(self.handle.lib.nb_network_output, self.output_size, device)

    def logits(self, device=None):
        return self._fetch(self.handle.lib.nb_network_logits, self.logits_size, device)

    def layer_output(self, i, rows):
        info = self.layer_info(i)
        out = np.empty(info["size"] * rows, np.float32)
        self.handle.check(self.handle.lib.nb_network_layer_output(self.n, i, _ptr(out), MEM_HOST))
        return out

    def close(self):
        if self.n:
            self.handle.lib.nb_network_destroy(self.n)
            self.n = _VP()
