"""The C-ABI library loads on a CPU-only machine and exports every symbol that
include/*.h declares.  No compute call is made here."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = set()
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names |= set(re.findall(r"\b((?:b200|ggml_backend)_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_headers_declare_entry_points():
    names = declared_symbols()
    assert "ggml_backend_init" in names and "ggml_backend_score" in names
    assert "b200_mul_mat_q" in names and "b200_flash_attn" in names


def test_library_exports_every_declared_symbol(b200):
    if not b200.LIB_PATH.exists():
        pytest.fail(f"{b200.LIB_PATH} not built: run python -c 'import __graft_entry__ as g; g.build()'")
    lib = ctypes.CDLL(str(b200.LIB_PATH))
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(set(b200.EXPORTS)) == declared_symbols()


def test_plugin_registry_without_gpu(b200):
    """ggml_backend_init must return a registry object (possibly with zero devices), never crash."""
    lib = ctypes.CDLL(str(b200.LIB_PATH))
    lib.ggml_backend_init.restype = ctypes.c_void_p
    reg = lib.ggml_backend_init()
    assert reg
    api_version = ctypes.cast(reg, ctypes.POINTER(ctypes.c_int))[0]
    assert api_version == 1          # GGML_BACKEND_API_VERSION, ggml/src/ggml-backend-impl.h:11
    assert lib.ggml_backend_score() in (0, 100)
    assert lib.b200_device_count() >= 0


def test_row_size_matches_oracle(b200, oracle):
    for qt in oracle.QUANT_TYPES:
        for k in (256, 4096, 14336):
            assert b200.row_size(qt, k) == oracle.row_size(qt, k)


def test_compute_fails_loudly_without_gpu(b200):
    import numpy as np
    if b200.device_count() > 0:
        pytest.skip("a B200 is present")
    with pytest.raises(b200.B200Error):
        b200.mul_mat_q("q4_0", np.zeros((8, 18 * 8), np.uint8), np.zeros((1, 256), np.float32))
