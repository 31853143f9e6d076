"""Back-to-back forward passes (the way the benchmark drives the library), each case in a child process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name,batch", [("vgg16", 32), ("lstm2", 16), ("alexnet", 16)])
def test_back_to_back_forwards_are_identical(name, batch):
    """Kernels of consecutive forward passes queue up behind one another with no host synchronisation in between:
    every pass must reproduce the first one bit for bit.  A failing child is reported, never run again."""
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, os.path.join(ROOT, "tests", "back_to_back_child.py"), name, str(batch), "6"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    if r.returncode == 0 and r.stdout.strip().endswith("OK"):
        return
    tail = (r.stdout + r.stderr).strip().splitlines()[-3:]
    pytest.fail(f"child exited {r.returncode}: {tail}")
