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


CASES = {"toy_convnet": (toy_convnet, 101), "shortcuts": (shortcut_net, 102), "tiny_lstm": (tiny_lstm, 103),
         "lstm_bn": (lstm_bn_net, 104)}


def main():
    out_dir = Path(__file__).resolve().parent
    for name, (make, seed) in CASES.items():
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
