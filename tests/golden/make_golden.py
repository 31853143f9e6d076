"""Generates the golden vectors under tests/golden/ by running the UNMODIFIED
reference CPU path (the binaries compiled from the reference sources by
oracle/Makefile into oracle/_ref/) on small seeded networks.

    make -C oracle ref && python tests/golden/make_golden.py

Each .npz holds the network.cfg text, the weight stream, the input batch and
every layer's output_data as written by the reference (both its in-tree GEMM
build, `custom`, and its OpenBLAS build, `oblas`).  The reference ships no test
vectors of its own; these pin the CPU restatement in oracle/nebula_oracle.c to
the reference's actual outputs and travel to machines without the reference.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import oracle as O  # noqa: E402
from tests.nets import tiny_lstm, toy_convnet  # noqa: E402
from nebula_b200.workloads import NetBuilder  # noqa: E402


def shortcut_net():
    """Channel- and stride-mismatched shortcuts, default pool padding, every cheap activation."""
    b = NetBuilder("shortcuts", 2, 4, 12, 12, bias_init="bias_n01")
    b.conv(8, 3, 1, 1, "relu").conv(8, 3, 1, 1, "ramp", bn=True).conv(16, 3, 2, 1, "plse").shortcut(2, "relie")
    b.maxpool(3, 2).conv(6, 1, 1, 0, "loggy").conv(6, 3, 1, 1, "elu").shortcut(2, "linear").avgpool(3, 3)
    b.connected(12, "stair").connected(5, "hardtan").connected(4, "lhtan").softmax()
    return b.build("normal")


def lstm_bn_net():
    b = NetBuilder("lstm_bn", 3, input_size=10, time_steps=4, bias_init="bias_n01")
    b.lstm(6, bn=True, bound=0.4).lstm(5, bound=0.4).connected(7, "linear", init="uniform", bound=0.4).softmax()
    return b.build("normal")


def rnn_net():
    """Two vanilla RNN layers (the second batch-normalised) and a projection: rnn_layer.cc:91-141."""
    b = NetBuilder("rnn", 3, input_size=12, time_steps=5, bias_init="bias_n01")
    b.rnn(8, "tanh", bound=0.4).rnn(6, "leaky", bn=True, bound=0.4).connected(7, "linear", init="uniform", bound=0.4).softmax()
    return b.build("normal")


def lstm_act_net():
    """LSTM whose eight gate layers carry a non-linear section activation (lstm_layer.cc:252-282)."""
    b = NetBuilder("lstm_act", 3, input_size=10, time_steps=4, bias_init="bias_n01")
    b.lstm(6, act="tanh", bound=0.4).lstm(5, act="leaky", bn=True, bound=0.4)
    b.connected(7, "linear", init="uniform", bound=0.4).softmax()
    return b.build("normal")


def dbn_net():
    """[rbm] layers at inference (rbm_layer.cc:345-374) and a linear classifier, as in benchmarks/dbn_*/network.cfg."""
    b = NetBuilder("dbn", 4, 3, 6, 5, bias_init="bias_n01")
    b.rbm(20, "logistic").rbm(12, "logistic").rbm(8, "tanh").connected(5, "linear").softmax()
    return b.build()


CASES = {"toy_convnet": (toy_convnet, 101), "shortcuts": (shortcut_net, 102), "tiny_lstm": (tiny_lstm, 103),
         "lstm_bn": (lstm_bn_net, 104), "rnn": (rnn_net, 105), "lstm_act": (lstm_act_net, 106), "dbn": (dbn_net, 107)}


def main():
    out_dir = Path(__file__).resolve().parent
    only = set(sys.argv[1:])
    for name, (make, seed) in CASES.items():
        if only and name not in only:
            continue
        wl = make()
        w = wl.make_weights(seed)
        x = wl.make_input(seed + 1000)
        blobs = {"cfg": np.array(wl.cfg), "weights": w, "input": x, "recurrent": np.array(wl.recurrent)}
        for flavour in ("custom", "oblas"):
            outs, info = O.run_reference(wl.cfg, w, x, recurrent=wl.recurrent, flavour=flavour, dump_all=True, threads=4)
            for i, o in enumerate(outs):
                blobs[f"{flavour}_layer_{i:02d}"] = o
        np.savez_compressed(out_dir / f"{name}.npz", **blobs)
        print(name, "layers", len(outs), "weights", w.size, "bytes", (out_dir / f"{name}.npz").stat().st_size)


if __name__ == "__main__":
    main()
