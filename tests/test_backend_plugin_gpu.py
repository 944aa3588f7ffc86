"""Drop-in check: the reference's own, unmodified test-backend-ops binary (built by
oracle/ref.mk) loads libggml-b200.so through GGML_BACKEND_PATH and compares every
op the device claims with the reference CPU backend."""
import os
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"


def run_tbo(*args, timeout=900):
    if not (REF / "test-backend-ops").exists():
        pytest.skip("oracle/_ref/test-backend-ops not built (make -f oracle/ref.mk core)")
    env = dict(os.environ, GGML_BACKEND_PATH=str(ROOT / "llama.cpp_b200" / "lib" / "libggml-b200.so"))
    return subprocess.run([str(REF / "test-backend-ops"), *args], cwd=REF, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("op", ["MUL_MAT", "MUL_MAT_ID", "FLASH_ATTN_EXT", "GET_ROWS", "CPY", "RMS_NORM", "ROPE", "SOFT_MAX",
                                "ADD", "MUL", "SILU", "CONT", "DUP", "SCALE"])
def test_reference_test_backend_ops(op):
    r = run_tbo("test", "-b", "B200_0", "-o", op)
    out = r.stdout + r.stderr
    assert "Backend B200_0" in out, out[-2000:]
    fails = [l for l in out.splitlines() if "FAIL" in l]
    assert r.returncode == 0 and not fails, "\n".join(fails[:20]) + out[-1500:]
    ran = [l for l in out.splitlines() if l.strip().startswith(op + "(") and "OK" in l]
    assert ran, f"no {op} case ran on the device"
