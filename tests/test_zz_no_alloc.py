"""The allocation-free connected-layer entry point (nb_fc_forward_static) against
the plan-based one.  Its scratch is one array shared by all calls, so the test
makes two calls in a row with different shapes and checks both: what the first
call left in the array must not leak into the second.  Kept in a file that
pytest collects last."""
import numpy as np
import pytest

from tests.util import TOL, rel_err

pytestmark = pytest.mark.gpu


def _pair(handle, batch, inputs, outputs, act, seed):
    import torch
    from nebula_b200 import api
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((batch, inputs), dtype=np.float32)).cuda()
    w = torch.from_numpy((rng.standard_normal((outputs, inputs)) / np.sqrt(inputs)).astype(np.float32)).cuda()
    b = torch.from_numpy((0.1 * rng.standard_normal(outputs)).astype(np.float32)).cuda()
    plan = api.Connected(handle, batch, inputs, outputs, False, act)
    plan.set_weights(w, b)
    want = plan.forward(x).cpu().numpy()
    got = handle.fc_forward_static(x, w, b, act).cpu().numpy()
    handle.synchronize()
    plan.close()
    return got, want


@pytest.mark.parametrize("mode", ["tf32", "tf32x3", "fp32"])
def test_static_entry_matches_plan_entry_twice_in_a_row(mode):
    from nebula_b200 import api
    handle = api.Handle(0, mode)          # own handle: the test also has to pass alone in a fresh process
    try:
        # first a large call that fills most of the array, then a smaller one with another shape
        for batch, inputs, outputs, act, seed in ((256, 2048, 1000, "relu", 1), (33, 96, 130, "leaky", 2)):
            got, want = _pair(handle, batch, inputs, outputs, act, seed)
            assert np.isfinite(got).all()
            assert rel_err(got, want) <= TOL[mode], f"{mode} {batch}x{inputs}x{outputs}: {rel_err(got, want):.3e}"
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
