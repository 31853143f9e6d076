"""Network-level driver for the CPU restatement in ``nebula_oracle.c`` and a thin
runner for the compiled reference under ``oracle/_ref``.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
bench's CPU-baseline leg.  Nothing in the product package may import it.

The cfg reader restates the reference's parser (common/config.cc:44-75: every
space is stripped, ``#`` lines and blank lines are skipped, ``[name]`` opens a
section, keys and values are lower-cased) and the layer shape rules
(convolutional_layer.cc:119-153, pooling_layer.cc:40-63, connected_layer.cc:98-112,
shortcut_layer.cc:32-50, lstm_layer.cc:84-128).  The weight reader follows the
weight-file order (network.cc:99-122 and each layer's init_weight).
"""
from __future__ import annotations

import ctypes
import json
import os
import subprocess
import tempfile
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None

ACT = {"elu": 1, "hardtan": 2, "leaky": 3, "lhtan": 4, "linear": 5, "loggy": 6, "logistic": 7,
       "plse": 8, "ramp": 9, "relie": 10, "relu": 11, "stair": 12, "tanh": 13}


class _Blob(ctypes.Structure):
    _fields_ = [(n, ctypes.POINTER(ctypes.c_float)) for n in ("bias", "w", "scale", "mean", "var")]


def build(force: bool = False) -> Path:
    """Compiles the C restatement (and, when the reference tree is present, the
    reference binaries) with the Makefile beside this file."""
    so = HERE / "libnebula_oracle.so"
    if force or not so.exists() or so.stat().st_mtime < (HERE / "nebula_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "restate"], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(build()))
        _LIB.nbo_set_threads(min(os.cpu_count() or 1, 64))
    return _LIB


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ----------------------------------------------------------------- operators
def conv_forward(x, w, bias, k, stride, pad, act, bn=None):
    """x [B,C,H,W], w [F,C,k,k]; bn = (scale, mean, var) or None."""
    x, w, bias = _f32(x), _f32(w), _f32(bias)
    B, C, H, W = x.shape
    F = w.shape[0]
    OH, OW = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    y = np.empty((B, F, OH, OW), np.float32)
    s, m, v = (_f32(t) for t in bn) if bn is not None else (None, None, None)
    lib().nbo_conv_forward(_fp(x), B, C, H, W, F, k, stride, pad, _fp(w), _fp(bias), _fp(s), _fp(m), _fp(v),
                           ACT[act], _fp(y))
    return y


def connected_forward(x, w, bias, act, bn=None):
    x, w, bias = _f32(x), _f32(w), _f32(bias)
    B = x.shape[0]
    x2 = x.reshape(B, -1)
    out, inp = w.shape
    assert x2.shape[1] == inp
    y = np.empty((B, out), np.float32)
    s, m, v = (_f32(t) for t in bn) if bn is not None else (None, None, None)
    lib().nbo_connected_forward(_fp(x2), B, inp, out, _fp(w), _fp(bias), _fp(s), _fp(m), _fp(v), ACT[act], _fp(y))
    return y


def pool_forward(x, k, stride, pad, is_max):
    x = _f32(x)
    B, C, H, W = x.shape
    OH, OW = (H + 2 * pad) // stride, (W + 2 * pad) // stride
    y = np.empty((B, C, OH, OW), np.float32)
    lib().nbo_pool_forward(_fp(x), B, C, H, W, k, stride, pad, int(is_max), _fp(y))
    return y


def shortcut_forward(prev, conn, act):
    prev, conn = _f32(prev), _f32(conn)
    B, Co, Ho, Wo = prev.shape
    _, Ci, Hi, Wi = conn.shape
    y = np.empty_like(prev)
    lib().nbo_shortcut_forward(_fp(prev), _fp(conn), B, Ci, Hi, Wi, Co, Ho, Wo, ACT[act], _fp(y))
    return y


def softmax_forward(x):
    x = _f32(x)
    B = x.shape[0]
    x2 = x.reshape(B, -1)
    y = np.empty_like(x2)
    lib().nbo_softmax_forward(_fp(x2), B, x2.shape[1], _fp(y))
    return y.reshape(x.shape)


def activate(x, act):
    y = _f32(x).copy()
    lib().nbo_activate(_fp(y), ctypes.c_long(y.size), ACT[act])
    return y


def lstm_forward(x, blobs, H, act="linear", has_bn=False):
    """x [T,B,in] time-major; blobs = 8 dicts (bias,w[,scale,mean,var]) in file
    order iW,fW,oW,cW,iU,fU,oU,cU.  Returns (out [T,B,H], cell [T,B,H])."""
    x = _f32(x)
    T, B, inp = x.shape
    keep = []
    arr = (_Blob * 8)()
    for i, b in enumerate(blobs):
        for name in ("bias", "w", "scale", "mean", "var"):
            a = _f32(b[name]) if b.get(name) is not None else None
            keep.append(a)
            setattr(arr[i], name, _fp(a))
    out = np.empty((T, B, H), np.float32)
    cell = np.empty((T, B, H), np.float32)
    lib().nbo_lstm_forward(_fp(x), T, B, inp, H, arr, int(has_bn), ACT[act], _fp(out), _fp(cell))
    return out, cell


def gemm(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc):
    """gemm<T> (common/gemm.h:111-147) on flat row-major buffers; returns the updated copy of C."""
    A, B, C = _f32(A).ravel(), _f32(B).ravel(), _f32(C).ravel().copy()
    lib().nbo_gemm(int(ta), int(tb), M, N, K, ctypes.c_float(alpha), _fp(A), lda, _fp(B), ldb, ctypes.c_float(beta), _fp(C), ldc)
    return C


def rnn_forward(x, blobs, H, act, has_bn=False):
    """x [T,B,in] time-major; blobs = 3 dicts in file order input, hidden, output gate.  Returns out [T,B,H]."""
    x = _f32(x)
    T, B, inp = x.shape
    keep = []
    arr = (_Blob * 3)()
    for i, b in enumerate(blobs):
        for name in ("bias", "w", "scale", "mean", "var"):
            a = _f32(b[name]) if b.get(name) is not None else None
            keep.append(a)
            setattr(arr[i], name, _fp(a))
    out = np.empty((T, B, H), np.float32)
    lib().nbo_rnn_forward(_fp(x), T, B, inp, H, arr, int(has_bn), ACT[act], _fp(out))
    return out


# ------------------------------------------------------------------- configs
@dataclass
class Section:
    name: str
    settings: dict = field(default_factory=dict)

    def get(self, key, default=None, cast=int):
        v = self.settings.get(key.lower())
        return default if v is None else cast(v)


def parse_cfg(text: str) -> list[Section]:
    """common/config.cc:44-75."""
    sections: list[Section] = []
    for line in text.splitlines():
        line = line.replace(" ", "")
        if not line or line[0] == "#":
            continue
        if line[0] == "[":
            sections.append(Section(line[1:-1]))
        else:
            if "=" not in line:
                raise ValueError(f"invalid config line: {line}")
            k, v = line.split("=", 1)
            # std::map::insert keeps the first value of a repeated key
            sections[-1].settings.setdefault(k.lower(), v.lower())
    return sections


@dataclass
class Layer:
    kind: str
    sec: Section
    out_shape: tuple            # (C,H,W) for spatial layers, (n,) for flat ones
    params: dict = field(default_factory=dict)


def _flat(shape):
    n = 1
    for d in shape:
        n *= d
    return n


def plan_network(text: str):
    """Returns (net settings, layers) with every layer's output shape, following
    each layer class's init()."""
    secs = parse_cfg(text)
    net = {}
    layers: list[Layer] = []
    for sec in secs:
        if sec.name == "net":
            net = dict(batch=sec.get("batch", 1), height=sec.get("height", 1), width=sec.get("width", 1),
                       channels=sec.get("channels", 1), input_size=sec.get("input_size", 0),
                       time_steps=sec.get("time_steps", 1))
            net["recurrent"] = "input_size" in sec.settings
            cur = (net["input_size"],) if net["recurrent"] else (net["channels"], net["height"], net["width"])
            continue
        if sec.name == "cost":
            continue
        prev = layers[-1].out_shape if layers else cur
        if sec.name == "convolutional":
            C, H, W = prev
            F, k = sec.get("filters", 1), sec.get("size", 1)
            s, p = sec.get("stride", 1), sec.get("padding", 0)
            out = (F, (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1)
            layers.append(Layer("convolutional", sec, out, dict(C=C, H=H, W=W, F=F, k=k, s=s, p=p,
                                                                 bn=sec.get("batch_normalize", 0),
                                                                 act=sec.get("activation", None, str))))
        elif sec.name == "connected":
            out = (sec.get("output", 0),)
            layers.append(Layer("connected", sec, out, dict(inp=_flat(prev), out=out[0],
                                                             bn=sec.get("batch_normalize", 0),
                                                             act=sec.get("activation", None, str))))
        elif sec.name in ("maxpool", "avgpool"):
            C, H, W = prev
            s = sec.get("stride", 1)
            k = sec.get("size", s)
            p = sec.get("padding", (k - 1) // 2)
            out = (C, (H + 2 * p) // s, (W + 2 * p) // s)
            layers.append(Layer(sec.name, sec, out, dict(k=k, s=s, p=p)))
        elif sec.name == "shortcut":
            hops = sec.get("hops", 0)
            layers.append(Layer("shortcut", sec, prev, dict(conn=len(layers) - hops,
                                                             act=sec.get("activation", None, str))))
        elif sec.name in ("dropout", "softmax"):
            layers.append(Layer(sec.name, sec, prev))
        elif sec.name == "lstm":
            out = (sec.get("output", 0),)
            layers.append(Layer("lstm", sec, out, dict(inp=_flat(prev), H=out[0], bn=sec.get("batch_normalize", 0),
                                                        act=sec.get("activation", None, str))))
        elif sec.name == "rnn":
            out = (sec.get("output", 0),)
            layers.append(Layer("rnn", sec, out, dict(inp=_flat(prev), H=out[0], bn=sec.get("batch_normalize", 0),
                                                       act=sec.get("activation", None, str))))
        elif sec.name == "rbm":
            # rbm_layer_t::forward is a connected layer on hidden_bias (rbm_layer.cc:345-374); no batch-norm
            out = (sec.get("output", 0),)
            layers.append(Layer("connected", sec, out, dict(inp=_flat(prev), out=out[0], bn=0,
                                                             act=sec.get("activation", None, str))))
        else:
            raise ValueError(f"unknown layer type {sec.name}")
    return net, layers


def weight_count(layers) -> int:
    n = 0
    for l in layers:
        p = l.params
        if l.kind == "convolutional":
            n += p["F"] + p["F"] * p["C"] * p["k"] ** 2 + (3 * p["F"] if p["bn"] else 0)
        elif l.kind == "connected":
            n += p["out"] + p["out"] * p["inp"] + (3 * p["out"] if p["bn"] else 0)
        elif l.kind == "lstm":
            for g in range(8):
                gin = p["H"] if g < 4 else p["inp"]
                n += p["H"] + p["H"] * gin + (3 * p["H"] if p["bn"] else 0)
        elif l.kind == "rnn":
            for gin in (p["inp"], p["H"], p["H"]):
                n += p["H"] + p["H"] * gin + (3 * p["H"] if p["bn"] else 0)
    return n


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = np.frombuffer(buf, dtype="<f4") if not isinstance(buf, np.ndarray) else buf, 0

    def take(self, n):
        if self.pos + n > self.buf.size:
            raise ValueError("weight stream too short")
        a = self.buf[self.pos:self.pos + n]
        self.pos += n
        return a

    def fc(self, out, inp, bn):
        b = dict(bias=self.take(out), w=self.take(out * inp).reshape(out, inp))
        if bn:
            b.update(scale=self.take(out), mean=self.take(out), var=self.take(out))
        return b


def forward_network(cfg_text: str, weights, x, batch=None, keep_all=False):
    """Runs the restated network on x (NCHW [B,C,H,W], or time-major [T,B,in]
    for recurrent nets).  Returns the list of layer outputs (all of them if
    keep_all, else only the last one)."""
    net, layers = plan_network(cfg_text)
    rd = _Reader(weights)
    outs = []
    cur = _f32(x)
    for l in layers:
        p = l.params
        if l.kind == "convolutional":
            bias = rd.take(p["F"])
            w = rd.take(p["F"] * p["C"] * p["k"] ** 2).reshape(p["F"], p["C"], p["k"], p["k"])
            bn = (rd.take(p["F"]), rd.take(p["F"]), rd.take(p["F"])) if p["bn"] else None
            cur = conv_forward(cur, w, bias, p["k"], p["s"], p["p"], p["act"], bn)
        elif l.kind == "connected":
            b = rd.fc(p["out"], p["inp"], p["bn"])
            lead = cur.shape[:2] if net["recurrent"] else cur.shape[:1]
            rows = cur.reshape(int(np.prod(lead)), -1)
            cur = connected_forward(rows, b["w"], b["bias"], p["act"],
                                    (b["scale"], b["mean"], b["var"]) if p["bn"] else None).reshape(*lead, p["out"])
        elif l.kind in ("maxpool", "avgpool"):
            cur = pool_forward(cur, p["k"], p["s"], p["p"], l.kind == "maxpool")
        elif l.kind == "shortcut":
            cur = shortcut_forward(cur, outs[p["conn"]], p["act"])
        elif l.kind == "dropout":
            pass
        elif l.kind == "softmax":
            cur = softmax_forward(cur.reshape(-1, cur.shape[-1]) if net["recurrent"] else cur).reshape(cur.shape)
        elif l.kind == "lstm":
            blobs = [rd.fc(p["H"], p["H"] if g < 4 else p["inp"], p["bn"]) for g in range(8)]
            cur, _ = lstm_forward(cur, blobs, p["H"], p["act"], bool(p["bn"]))
        elif l.kind == "rnn":
            blobs = [rd.fc(p["H"], gin, p["bn"]) for gin in (p["inp"], p["H"], p["H"])]
            cur = rnn_forward(cur, blobs, p["H"], p["act"], bool(p["bn"]))
        outs.append(cur)
    return outs if keep_all else outs[-1:]


# -------------------------------------------------------- compiled reference
def ref_binary(flavour: str = "oblas") -> Path | None:
    """Path of the compiled reference (``oblas`` = its default OpenBLAS build,
    ``custom`` = its in-tree GEMM), or None when it has not been built."""
    p = HERE / "_ref" / f"nebula_ref_{flavour}"
    return p if p.exists() else None


def run_reference(cfg_text: str, weights: np.ndarray, x: np.ndarray, *, recurrent=False, flavour="oblas",
                  threads=None, reps=1, out_layer=-1, dump_all=False, batch=None):
    """Executes the compiled reference on the given bytes.  Returns
    (output array flat, info dict) or, with dump_all, (list of flat arrays, info)."""
    exe = ref_binary(flavour)
    if exe is None:
        raise FileNotFoundError(f"oracle/_ref/nebula_ref_{flavour} is not built (make -C oracle ref)")
    with tempfile.TemporaryDirectory() as d:
        d = Path(d)
        (d / "net.cfg").write_text(cfg_text)
        _f32(x).tofile(d / "in.bin")
        _f32(weights).tofile(d / "w.wgh")
        cmd = [str(exe), "--cfg", str(d / "net.cfg"), "--input", str(d / "in.bin"), "--weights", str(d / "w.wgh"),
               "--out", str(d / "out.bin"), "--out-layer", str(out_layer), "--reps", str(reps),
               "--threads", str(threads or min(os.cpu_count() or 1, 64))]
        if recurrent:
            cmd.append("--recurrent")
        if batch:
            cmd += ["--batch", str(batch)]
        if dump_all:
            (d / "dump").mkdir()
            cmd += ["--dump-dir", str(d / "dump")]
        r = subprocess.run(cmd, check=True, capture_output=True, text=True)
        info = json.loads(r.stdout.strip().splitlines()[-1])
        if dump_all:
            return [np.fromfile(f, np.float32) for f in sorted((d / "dump").glob("layer_*.bin"))], info
        return np.fromfile(d / "out.bin", np.float32), info
