"""Back-to-back forward passes (the way the benchmark drives the library), each case in a child process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


KNOWN = pytest.mark.xfail(strict=False, reason="open issue: on some boxes of the pool this case ends in an illegal-address "
                         "fault (about 4 boxes in 10; clean on the others with the same binaries); the failure "
                         "text names the launch and the device")


@pytest.mark.parametrize("name,batch", [("vgg16", 32), pytest.param("resnet50", 32, marks=KNOWN), ("lstm2", 16),
                                        ("alexnet", 16)])
def test_back_to_back_forwards_are_identical(name, batch):
    """Kernels of consecutive forward passes queue up behind one another with no host synchronisation in between:
    every pass must reproduce the first one bit for bit."""
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, os.path.join(ROOT, "tests", "back_to_back_child.py"), name, str(batch), "6"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    if r.returncode == 0 and r.stdout.strip().endswith("OK"):
        return
    tail = (r.stdout + r.stderr).strip().splitlines()[-3:]
    # say where: the same passes with a synchronisation after every launch name the failing kernel and its geometry
    r2 = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT,
                        env=dict(env, NEBULA_B200_SYNC_LAUNCHES="1"))
    tail2 = (r2.stdout + r2.stderr).strip().splitlines()[-2:]
    try:
        smi = subprocess.run(["nvidia-smi", "--query-gpu=name,driver_version,vbios_version,memory.used,clocks.sm,power.limit",
                              "--format=csv,noheader"], capture_output=True, text=True, timeout=30).stdout.strip()
    except (OSError, subprocess.SubprocessError):
        smi = "nvidia-smi unavailable"
    pytest.fail(f"child exited {r.returncode}: {tail}; with a synchronisation after every launch it exited "
                f"{r2.returncode}: {tail2}; device: {smi}")
