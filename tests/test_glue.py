"""The Nebula-side glue (glue/nebula_forward_glue.cu) compiles against the reference's own, unmodified headers:
every field of layer_t / network_t and of the layer classes that it reads is checked by the compiler.  Needs the
reference tree (the REF variable of oracle/Makefile); skipped on machines without it."""
import re
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _ref_dir():
    m = re.search(r"^REF\s*\?=\s*(\S+)", (ROOT / "oracle" / "Makefile").read_text(), re.M)
    return Path(m.group(1)) if m else None


@pytest.mark.skipif(shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists(), reason="no nvcc")
def test_glue_compiles_against_the_reference_headers(tmp_path):
    ref = _ref_dir()
    if ref is None or not (ref / "models" / "layers" / "layer.h").exists():
        pytest.skip("reference tree not present")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-c", "-std=c++14", "-DGPU_ENABLED", "-DNEBULA_B200", f"-I{ROOT / 'include'}", f"-I{ref / 'common'}",
           f"-I{ref / 'models' / 'layers'}", f"-I{ref / 'models' / 'networks'}", "-gencode", "arch=compute_100a,code=sm_100a",
           str(ROOT / "glue" / "nebula_forward_glue.cu"), "-o", str(tmp_path / "glue.o")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    # the object defines the forward methods it claims to replace
    nm = subprocess.run(["nm", "-C", str(tmp_path / "glue.o")], capture_output=True, text=True).stdout
    for cls in ("convolutional_layer_t", "connected_layer_t", "pooling_layer_t", "shortcut_layer_t", "softmax_layer_t",
                "lstm_layer_t", "rnn_layer_t", "rbm_layer_t"):
        assert re.search(rf" T nebula::{cls}::_forward_\(", nm), f"{cls}::_forward_ is not defined by the glue"
