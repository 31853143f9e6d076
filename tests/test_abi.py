"""The C-ABI library loads and exports every symbol include/nebula_b200.h declares
(no compute calls: this runs without a GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib_path():
    from nebula_b200 import build
    return build.build()


def _declared():
    text = (ROOT / "include" / "nebula_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = _declared()
    for must in ("nb_create", "nb_conv2d_forward", "nb_fc_forward", "nb_pool_forward", "nb_shortcut_forward",
                 "nb_lstm_forward", "nb_softmax_forward", "nb_network_forward", "nb_network_load_weights"):
        assert must in names
    assert len(names) >= 40


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_python_binding_covers_the_header(lib_path):
    from nebula_b200 import api
    assert sorted(api.SIGNATURES) == _declared()
    api.load_library(lib_path)


def test_missing_library_fails_loudly(tmp_path):
    from nebula_b200 import api
    with pytest.raises(FileNotFoundError):
        api.load_library(tmp_path / "libnebula_b200.so")


def test_no_gpu_means_error_not_fallback(lib_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = ctypes.CDLL(str(lib_path))
    h = ctypes.c_void_p()
    rc = lib.nb_create(0, ctypes.byref(h))
    assert rc != 0 and not h.value


def test_product_never_touches_the_oracle():
    """Only tests, the smoke check and the bench's CPU-baseline leg may use oracle/."""
    for path in list((ROOT / "nebula_b200").rglob("*.py")) + list((ROOT / "nebula_b200" / "csrc").glob("*")):
        if path.is_file():
            assert "oracle" not in path.read_text(errors="ignore"), f"{path} mentions the oracle"
