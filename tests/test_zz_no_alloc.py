"""The allocation-free connected-layer entry point (nb_fc_forward_static) against
the plan-based one and against the CPU oracle.  Its scratch is one array shared
by all calls, so the test makes two calls in a row with different shapes and
checks both: what the first call left in the array must not leak into the
second.  It also checks the claim itself: the device's free memory is the same
before and after the calls.  Kept in a file that pytest collects last."""
import numpy as np
import pytest

from tests.util import TOL, rel_err

pytestmark = pytest.mark.gpu


def _case(batch, inputs, outputs, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, inputs), dtype=np.float32)
    w = (rng.standard_normal((outputs, inputs)) / np.sqrt(inputs)).astype(np.float32)
    b = (0.1 * rng.standard_normal(outputs)).astype(np.float32)
    return x, w, b


@pytest.mark.parametrize("mode", ["tf32", "tf32x3", "fp32"])
def test_static_entry_matches_plan_entry_and_oracle_twice_in_a_row(mode):
    import torch
    from nebula_b200 import api
    from oracle import oracle as O
    handle = api.Handle(0, mode)          # own handle: the test also has to pass alone in a fresh process
    try:
        # first a large call that fills most of the array, then a smaller one with another shape
        for batch, inputs, outputs, act, seed in ((256, 2048, 700, "relu", 1), (33, 96, 130, "leaky", 2)):
            x, w, b = _case(batch, inputs, outputs, seed)
            xd, wd, bd = (torch.from_numpy(t).cuda() for t in (x, w, b))
            plan = api.Connected(handle, batch, inputs, outputs, False, act)
            plan.set_weights(wd, bd)
            want = plan.forward(xd).cpu().numpy()
            y = torch.empty((batch, outputs), device="cuda", dtype=torch.float32)
            handle.fc_forward_static(xd, wd, bd, act, out=y)        # first use on this device: looks the array up
            torch.cuda.synchronize()
            free0, _ = torch.cuda.mem_get_info()
            for _ in range(2):
                handle.fc_forward_static(xd, wd, bd, act, out=y)
            handle.synchronize()
            free1, _ = torch.cuda.mem_get_info()
            assert free1 == free0, f"device free memory changed by {free0 - free1} bytes across the static calls"
            got = y.cpu().numpy()
            ref = O.connected_forward(x, w, b, act)
            assert np.isfinite(got).all()
            assert rel_err(got, want) <= TOL[mode], f"{mode} {batch}x{inputs}x{outputs} vs plan: {rel_err(got, want):.3e}"
            assert rel_err(got, ref) <= TOL[mode], f"{mode} {batch}x{inputs}x{outputs} vs oracle: {rel_err(got, ref):.3e}"
            plan.close()
    finally:
        handle.close()


def test_static_entry_rejects_sizes_beyond_its_array():
    import torch
    from nebula_b200 import api
    handle = api.Handle(0, "tf32")
    try:
        x = torch.zeros(8, 4096, device="cuda")
        w = torch.zeros(2048, 4096, device="cuda")       # 8 Mi floats of weights alone
        b = torch.zeros(2048, device="cuda")
        with pytest.raises(api.NebulaError) as e:
            handle.fc_forward_static(x, w, b, "linear")
        assert e.value.code == 1 and "scratch" in str(e.value)
    finally:
        handle.close()
