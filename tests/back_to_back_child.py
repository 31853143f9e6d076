"""Child process of tests/test_gpu_stress.py: queues forward passes of one benchmark network with no host
synchronisation in between and compares the last pass with the first, bit for bit.  Runs in its own process so
that a device fault here cannot poison the CUDA context of the test session.  Prints one line: OK, or what differed."""
import sys

import numpy as np


def main():
    import torch
    from nebula_b200 import api, workloads
    name, batch, passes = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    kw = {"time_steps": 16} if name == "lstm2" else {}
    wl = workloads.WORKLOADS[name](batch=batch, **kw)
    handle = api.Handle(0, "tf32")
    net = api.Network(handle, wl.cfg)
    net.load_weights(wl.make_weights(4000))
    x = torch.from_numpy(wl.make_input(4001)).cuda()
    net.forward(x)
    handle.synchronize()
    first = net.logits().copy()
    if not np.isfinite(first).all():
        print("non-finite logits in the first pass")
        return 1
    for _ in range(passes):          # queued without waiting
        net.forward(x)
    handle.synchronize()
    again = net.logits()
    diff = first != again
    if diff.any():
        print(f"{int(diff.sum())} of {diff.size} logits changed, max |d| {np.abs(first - again).max():.3e}")
        return 1
    print("OK")
    return 0


if __name__ == "__main__":
    sys.exit(main())
